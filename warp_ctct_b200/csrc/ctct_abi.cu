// extern "C" entry points of libctct_b200.so (declared in include/ctct_b200.h): argument
// checks, workspace carving and kernel launches.  Nothing here allocates or synchronises.
#include "../../include/ctct_b200.h"

#include <cstdio>

#include "common.cuh"
#include "gather.cuh"
#include "grad.cuh"
#include "lattice.cuh"

using namespace ctct;

namespace {

thread_local char g_last_cuda_error[256] = "";

int check_launch(const char *what) {
    const cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) return CTCT_OK;
    snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s", what, cudaGetErrorString(err));
    return CTCT_ERR_LAUNCH;
}

// ---- optional event recorder (benchmarks only) ----
struct Profiler {
    cudaEvent_t *ev = nullptr;  // 4 per call
    int *kind = nullptr;
    int cap = 0, used = 0;
};
thread_local Profiler g_prof;

// returns the 4 events of the next call slot, or nullptr when profiling is off / full
cudaEvent_t *prof_slot(int kind) {
    if (!g_prof.ev || g_prof.used >= g_prof.cap) return nullptr;
    g_prof.kind[g_prof.used] = kind;
    return g_prof.ev + 4 * (g_prof.used++);
}
inline void prof_mark(cudaEvent_t *slot, int i, cudaStream_t st) {
    if (slot) cudaEventRecord(slot[i], st);
}

int sm_count() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms > 0 ? sms : 148;
}

// contexts per lane (C) and warps per direction (W) for a given number of contexts
struct LatCfg {
    int C, W, NL;
};
bool lattice_config(int64_t U1, LatCfg *cfg) {
    if (U1 < 1 || U1 > 8192) return false;
    int C, W = 1;
    if (U1 <= 32) C = 1;
    else if (U1 <= 64) C = 2;
    else if (U1 <= 96) C = 3;
    else if (U1 <= 128) C = 4;
    else if (U1 <= 160) C = 5;
    else if (U1 <= 192) C = 6;
    else {
        C = 8;
        const int need = static_cast<int>((U1 + 255) / 256);
        while (W < need) W *= 2;
    }
    cfg->C = C;
    cfg->W = W;
    cfg->NL = static_cast<int>(pad4((U1 + C - 1) / C));
    return true;
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

struct WsLayout {
    size_t G, TAB, OFF, LLF, LLI, total;
    int U1p;
    LatCfg cfg;
};
bool ws_layout(int64_t N, int64_t T, int64_t U1, int want_grad, WsLayout *w) {
    if (!lattice_config(U1, &w->cfg)) return false;
    w->U1p = static_cast<int>(pad4(U1));
    const size_t rows = static_cast<size_t>(N) * static_cast<size_t>(T);
    size_t o = 0;
    w->G = o;
    o = align256(o + rows * 3 * w->U1p * sizeof(float));
    w->TAB = o;
    if (want_grad) o = align256(o + rows * 4 * w->U1p * sizeof(float));
    w->OFF = o;
    if (want_grad) o = align256(o + rows * 2 * w->cfg.NL * sizeof(int));
    w->LLF = o;
    o = align256(o + static_cast<size_t>(N) * 2 * sizeof(float));
    w->LLI = o;
    o = align256(o + static_cast<size_t>(N) * 2 * sizeof(int));
    w->total = o;
    return true;
}

bool dims_ok(int64_t N, int64_t T, int64_t U1) {
    return N >= 0 && T >= 0 && U1 >= 1 && N <= 65535 && T * U1 < (int64_t(1) << 31) &&
           N * T * 3 * pad4(U1) < (int64_t(1) << 40);
}

template <int C, int W>
int launch_lattice_inst(const LatticeArgs &a, int N, size_t smem, cudaStream_t st) {
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(k_lattice<C, W>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)) != cudaSuccess)
            return check_launch("lattice smem attribute");
    }
    dim3 grid(N, a.beta_only ? 1 : 2);
    k_lattice<C, W><<<grid, W * 32, smem, st>>>(a);
    return check_launch("lattice");
}

int launch_lattice(LatticeArgs a, const LatCfg &cfg, int N, cudaStream_t st) {
    if (N == 0) return CTCT_OK;
    const size_t rowbytes = static_cast<size_t>(3) * a.U1p * sizeof(float);
    int F = static_cast<int>((48 * 1024) / rowbytes);
    F = F < 1 ? 1 : (F > 16 ? 16 : F);
    a.F = F;
    const size_t smem = 2 * static_cast<size_t>(F) * rowbytes + 4 * cfg.W * sizeof(float);
    if (smem > 220 * 1024) return CTCT_ERR_UNSUPPORTED;
#define LAT(Cv, Wv) \
    if (cfg.C == Cv && cfg.W == Wv) return launch_lattice_inst<Cv, Wv>(a, N, smem, st);
    LAT(1, 1) LAT(2, 1) LAT(3, 1) LAT(4, 1) LAT(5, 1) LAT(6, 1) LAT(8, 1)
    LAT(8, 2) LAT(8, 4) LAT(8, 8) LAT(8, 16) LAT(8, 32)
#undef LAT
    return CTCT_ERR_UNSUPPORTED;
}

template <typename InT>
int launch_gather_t(const void *lp, const int *ys, const int *lx, const int *ly, float *out, int64_t N,
                    int64_t T, int64_t U1, int64_t V, bool internal, int valid_only, cudaStream_t st) {
    const int U1p = static_cast<int>(pad4(U1));
    const int64_t total = internal ? N * T * 3 * U1p : N * T * U1 * 3;
    if (total == 0) return CTCT_OK;
    const int64_t want = (total + 256 * 4 - 1) / (256 * 4);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    const int grid = static_cast<int>(want < cap ? want : cap);
    const InT *p = static_cast<const InT *>(lp);
    const bool small = total < (int64_t(1) << 31) - int64_t(grid) * 256 * 4;
    if (internal) {
        if (small)
            k_gather3<InT, unsigned, true><<<grid, 256, 0, st>>>(p, ys, lx, ly, out, (int)T, (int)U1, U1p, (int)V, (unsigned)total, valid_only);
        else
            k_gather3<InT, unsigned long long, true><<<grid, 256, 0, st>>>(p, ys, lx, ly, out, (int)T, (int)U1, U1p, (int)V, (unsigned long long)total, valid_only);
    } else {
        if (small)
            k_gather3<InT, unsigned, false><<<grid, 256, 0, st>>>(p, ys, lx, ly, out, (int)T, (int)U1, U1p, (int)V, (unsigned)total, valid_only);
        else
            k_gather3<InT, unsigned long long, false><<<grid, 256, 0, st>>>(p, ys, lx, ly, out, (int)T, (int)U1, U1p, (int)V, (unsigned long long)total, valid_only);
    }
    return check_launch("gather");
}

int launch_gather(const void *lp, int dtype, const int *ys, const int *lx, const int *ly, float *out, int64_t N,
                  int64_t T, int64_t U1, int64_t V, bool internal, int valid_only, cudaStream_t st) {
    switch (dtype) {
    case CTCT_F32: return launch_gather_t<float>(lp, ys, lx, ly, out, N, T, U1, V, internal, valid_only, st);
    case CTCT_F16: return launch_gather_t<__half>(lp, ys, lx, ly, out, N, T, U1, V, internal, valid_only, st);
    case CTCT_BF16: return launch_gather_t<__nv_bfloat16>(lp, ys, lx, ly, out, N, T, U1, V, internal, valid_only, st);
    }
    return CTCT_ERR_ARG;
}

int launch_fill_grad(const WsLayout &w, char *ws, const int *ys, const int *lx, const int *ly, float *out,
                     int ref_layout, int64_t N, int64_t T, int64_t U1, cudaStream_t st) {
    if (N == 0 || T == 0) return CTCT_OK;
    GradArgs g;
    g.G = reinterpret_cast<const float *>(ws + w.G);
    g.TAB = reinterpret_cast<const float *>(ws + w.TAB);
    g.OFF = reinterpret_cast<const int *>(ws + w.OFF);
    g.llf = reinterpret_cast<const float *>(ws + w.LLF);
    g.lli = reinterpret_cast<const int *>(ws + w.LLI);
    g.ys = ys;
    g.lx = lx;
    g.ly = ly;
    g.out = out;
    g.T = (int)T;
    g.U1 = (int)U1;
    g.U1p = w.U1p;
    g.NL = w.cfg.NL;
    g.C = w.cfg.C;
    g.ref_layout = ref_layout;
    const int cells = static_cast<int>(T * U1);
    dim3 grid((cells + 255) / 256, (unsigned)N);
    k_fill_grad<<<grid, 256, 0, st>>>(g);
    return check_launch("fill_grad");
}

LatticeArgs make_lattice_args(const WsLayout &w, char *ws, const int *ys, const int *lx, const int *ly,
                              float *costs, int64_t T, int64_t U1, int want_grad) {
    LatticeArgs a;
    a.G = reinterpret_cast<const float *>(ws + w.G);
    a.ys = ys;
    a.lx = lx;
    a.ly = ly;
    a.TAB = reinterpret_cast<float *>(ws + w.TAB);
    a.OFF = reinterpret_cast<int *>(ws + w.OFF);
    a.llf = reinterpret_cast<float *>(ws + w.LLF);
    a.lli = reinterpret_cast<int *>(ws + w.LLI);
    a.costs = costs;
    a.T = (int)T;
    a.U1 = (int)U1;
    a.U1p = w.U1p;
    a.NL = w.cfg.NL;
    a.F = 1;
    a.beta_only = want_grad ? 0 : 1;
    return a;
}

template <typename OutT>
int launch_scatter_t(const ScatterArgs &a, cudaStream_t st) {
    if (a.rows == 0 || a.V == 0) return CTCT_OK;
    constexpr int E = OutOps<OutT>::E;
    const bool vec = (a.V % E == 0) && (reinterpret_cast<uintptr_t>(a.out) % 16 == 0);
    const int64_t want = (a.rows + 7) / 8;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    const int grid = static_cast<int>(want < cap ? want : cap);
    if (vec)
        k_scatter_dense<OutT, true><<<grid, 256, 0, st>>>(a);
    else
        k_scatter_dense<OutT, false><<<grid, 256, 0, st>>>(a);
    return check_launch("scatter_dense");
}

}  // namespace

extern "C" {

int ctct_b200_abi_version(void) { return 1; }

const char *ctct_b200_strerror(int code) {
    switch (code) {
    case CTCT_OK: return "ok";
    case CTCT_ERR_ARG: return "invalid argument";
    case CTCT_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
    case CTCT_ERR_LAUNCH: return g_last_cuda_error[0] ? g_last_cuda_error : "CUDA launch failed";
    case CTCT_ERR_UNSUPPORTED: return "size not supported by the kernels";
    }
    return "unknown error";
}

int64_t ctct_b200_padded_contexts(int64_t U1) { return pad4(U1); }

size_t ctct_b200_grads3_elems(int64_t N, int64_t T, int64_t U1) {
    if (N < 0 || T < 0 || U1 < 1) return 0;
    return static_cast<size_t>(N) * T * 3 * pad4(U1);
}

size_t ctct_b200_workspace_bytes(int64_t N, int64_t T, int64_t U1, int want_grad) {
    WsLayout w;
    if (!dims_ok(N, T, U1) || !ws_layout(N, T, U1, want_grad, &w)) return 0;
    return w.total;
}

int ctct_b200_loss_forward(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                           const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int want_grad,
                           float *costs, float *grads3, void *workspace, size_t workspace_bytes, void *stream) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (dtype != CTCT_F32 && dtype != CTCT_F16 && dtype != CTCT_BF16) return CTCT_ERR_ARG;
    if (N == 0) return CTCT_OK;
    if (!log_probs || !lx || !ly || !costs || (U1 > 1 && !ys) || (want_grad && !grads3)) return CTCT_ERR_ARG;
    WsLayout w;
    if (!ws_layout(N, T, U1, want_grad, &w)) return CTCT_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < w.total || reinterpret_cast<uintptr_t>(workspace) % 256) return CTCT_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);

    cudaEvent_t *slot = prof_slot(0);
    prof_mark(slot, 0, st);
    int rc = launch_gather(log_probs, dtype, ys, lx, ly, reinterpret_cast<float *>(ws + w.G), N, T, U1, V, true, 1, st);
    if (rc) return rc;
    prof_mark(slot, 1, st);
    rc = launch_lattice(make_lattice_args(w, ws, ys, lx, ly, costs, T, U1, want_grad), w.cfg, (int)N, st);
    if (rc) return rc;
    prof_mark(slot, 2, st);
    if (want_grad) rc = launch_fill_grad(w, ws, ys, lx, ly, grads3, 0, N, T, U1, st);
    prof_mark(slot, 3, st);
    return rc;
}

int ctct_b200_loss_backward(const float *grads3, const float *grad_out, const int32_t *ys, const int32_t *lx,
                            const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int dtype,
                            void *dense, void *stream) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (N == 0 || T == 0) return CTCT_OK;
    if (!grads3 || !grad_out || !lx || !ly || !dense || (U1 > 1 && !ys)) return CTCT_ERR_ARG;
    ScatterArgs a;
    a.GR = grads3;
    a.grad_out = grad_out;
    a.ys = ys;
    a.lx = lx;
    a.ly = ly;
    a.out = dense;
    a.T = (int)T;
    a.U1 = (int)U1;
    a.U1p = (int)pad4(U1);
    a.V = (int)V;
    a.rows = N * T * U1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype != CTCT_F32 && dtype != CTCT_F16 && dtype != CTCT_BF16) return CTCT_ERR_ARG;
    cudaEvent_t *slot = prof_slot(1);
    prof_mark(slot, 0, st);
    int rc = CTCT_ERR_ARG;
    switch (dtype) {
    case CTCT_F32: rc = launch_scatter_t<float>(a, st); break;
    case CTCT_F16: rc = launch_scatter_t<__half>(a, st); break;
    case CTCT_BF16: rc = launch_scatter_t<__nv_bfloat16>(a, st); break;
    }
    prof_mark(slot, 1, st);
    return rc;
}

int ctct_b200_gather(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                     int64_t N, int64_t T, int64_t U1, int64_t V, int valid_only, float *gathered, void *stream) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (N == 0 || T == 0) return CTCT_OK;
    if (!log_probs || !gathered || (U1 > 1 && !ys) || (valid_only && (!lx || !ly))) return CTCT_ERR_ARG;
    return launch_gather(log_probs, dtype, ys, lx, ly, gathered, N, T, U1, V, false, valid_only ? 1 : 0,
                         static_cast<cudaStream_t>(stream));
}

int ctct_b200_gathered_forward(const float *gathered, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                               int64_t N, int64_t T, int64_t U1, int want_grad, float *costs, float *grads,
                               void *workspace, size_t workspace_bytes, void *stream) {
    if (!dims_ok(N, T, U1)) return CTCT_ERR_ARG;
    if (N == 0) return CTCT_OK;
    if (!gathered || !lx || !ly || !costs || (U1 > 1 && !ys) || (want_grad && !grads)) return CTCT_ERR_ARG;
    WsLayout w;
    if (!ws_layout(N, T, U1, want_grad, &w)) return CTCT_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < w.total || reinterpret_cast<uintptr_t>(workspace) % 256) return CTCT_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);
    const int64_t total = N * T * 3 * w.U1p;
    if (total > 0) {
        const int64_t want = (total + 255) / 256;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
        k_repack_gathered<<<static_cast<int>(want < cap ? want : cap), 256, 0, st>>>(
            gathered, lx, ly, reinterpret_cast<float *>(ws + w.G), (int)T, (int)U1, w.U1p, total);
        int rc = check_launch("repack");
        if (rc) return rc;
    }
    int rc = launch_lattice(make_lattice_args(w, ws, ys, lx, ly, costs, T, U1, want_grad), w.cfg, (int)N, st);
    if (rc) return rc;
    if (want_grad) rc = launch_fill_grad(w, ws, ys, lx, ly, grads, 1, N, T, U1, st);
    return rc;
}

int ctct_b200_export_tables(const void *workspace, size_t workspace_bytes, const int32_t *lx, const int32_t *ly,
                            int64_t N, int64_t T, int64_t U1, double *alpha, double *beta_next, double *ll_alpha,
                            double *ll_beta, void *stream) {
    if (!dims_ok(N, T, U1)) return CTCT_ERR_ARG;
    if (N == 0) return CTCT_OK;
    if (!lx || !ly || !alpha || !beta_next || !ll_alpha || !ll_beta) return CTCT_ERR_ARG;
    WsLayout w;
    if (!ws_layout(N, T, U1, 1, &w)) return CTCT_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < w.total) return CTCT_ERR_WORKSPACE;
    const char *ws = static_cast<const char *>(workspace);
    ExportArgs e;
    e.TAB = reinterpret_cast<const float *>(ws + w.TAB);
    e.OFF = reinterpret_cast<const int *>(ws + w.OFF);
    e.llf = reinterpret_cast<const float *>(ws + w.LLF);
    e.lli = reinterpret_cast<const int *>(ws + w.LLI);
    e.lx = lx;
    e.ly = ly;
    e.alpha = alpha;
    e.beta_next = beta_next;
    e.ll_alpha = ll_alpha;
    e.ll_beta = ll_beta;
    e.T = (int)T;
    e.U1 = (int)U1;
    e.U1p = w.U1p;
    e.NL = w.cfg.NL;
    e.C = w.cfg.C;
    const int S = 2 * ((int)U1 - 1) + 1;
    const int64_t cells = T * S > 0 ? T * S : 1;
    dim3 grid((unsigned)((cells + 255) / 256), (unsigned)N);
    k_export_tables<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(e);
    return check_launch("export_tables");
}

int ctct_b200_profile_disable(void) {
    if (g_prof.ev) {
        for (int i = 0; i < 4 * g_prof.cap; ++i) cudaEventDestroy(g_prof.ev[i]);
        delete[] g_prof.ev;
        delete[] g_prof.kind;
    }
    g_prof = Profiler();
    return CTCT_OK;
}

int ctct_b200_profile_enable(int max_calls) {
    if (max_calls < 1 || max_calls > (1 << 20)) return CTCT_ERR_ARG;
    ctct_b200_profile_disable();
    g_prof.ev = new cudaEvent_t[4 * static_cast<size_t>(max_calls)];
    g_prof.kind = new int[max_calls];
    g_prof.cap = max_calls;
    for (int i = 0; i < 4 * max_calls; ++i)
        if (cudaEventCreate(&g_prof.ev[i]) != cudaSuccess) {
            g_prof.cap = i / 4;
            for (int j = 0; j < i; ++j) cudaEventDestroy(g_prof.ev[j]);
            delete[] g_prof.ev;
            delete[] g_prof.kind;
            g_prof = Profiler();
            return check_launch("profile events");
        }
    return CTCT_OK;
}

int ctct_b200_profile_read(float *ms, int *kind, int capacity) {
    if (!ms || !kind || capacity < 0) return CTCT_ERR_ARG;
    const int n = g_prof.used < capacity ? g_prof.used : capacity;
    for (int i = 0; i < n; ++i) {
        cudaEvent_t *e = g_prof.ev + 4 * i;
        const int pairs = g_prof.kind[i] == 0 ? 3 : 1;
        if (cudaEventSynchronize(e[pairs]) != cudaSuccess) return check_launch("profile sync");
        kind[i] = g_prof.kind[i];
        for (int k = 0; k < 3; ++k) {
            float t = 0.0f;
            if (k < pairs && cudaEventElapsedTime(&t, e[k], e[k + 1]) != cudaSuccess) return check_launch("profile elapsed");
            ms[4 * i + k] = t;
        }
        ms[4 * i + 3] = 0.0f;
    }
    g_prof.used = 0;
    return n;
}

}  // extern "C"
