// extern "C" entry points of libctct_b200.so (declared in include/ctct_b200.h): argument
// checks, workspace carving and kernel launches.  Nothing here allocates or synchronises.
#include "../../include/ctct_b200.h"

#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "gather.cuh"
#include "grad.cuh"
#include "lattice.cuh"
#include "logits.cuh"
#include "simple.cuh"
#include "logmm_tc.cuh"
#include "logmm_bwd_tc.cuh"
#include "logmm_bwd_fused.cuh"

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
// process-wide: autograd runs the backward call on a different host thread than the forward
Profiler g_prof;
std::mutex g_prof_mutex;

// returns the 4 events of the next call slot, or nullptr when profiling is off / full
cudaEvent_t *prof_slot(int kind) {
    if (!g_prof.ev) return nullptr;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    if (!g_prof.ev || g_prof.used >= g_prof.cap) return nullptr;
    g_prof.kind[g_prof.used] = kind;
    return g_prof.ev + 4 * (g_prof.used++);
}
inline void prof_mark(cudaEvent_t *slot, int i, cudaStream_t st) {
    if (slot) cudaEventRecord(slot[i], st);
}

// Launch with programmatic stream serialisation: the kernel may be set up, and start, while the
// kernel before it in the stream drains; it must call pdl_wait() before touching that kernel's output.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

int sm_count() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms > 0 ? sms : 148;
}

// Lattice slots (two per context) per thread and threads per CTA.  One warp handles 32 slots;
// with several warps, 2 lanes (1 when a thread holds more than one slot) of every warp are halo
// lanes, so a warp covers 30*C (31*C) slots.  One slot per thread up to 480 contexts.
struct LatCfg {
    int C, threads;
};
constexpr size_t kLatticeSmemLimit = 220 * 1024;
// Frames staged per chunk (F) and dynamic shared memory of a lattice CTA: two buffers of F rows of
// 16-byte records plus the exchange area between warps.
size_t lattice_smem(int64_t U1, int *F_out) {
    const size_t rowbytes = static_cast<size_t>(U1) * sizeof(float4);
    int F = static_cast<int>((48 * 1024) / rowbytes);
    const int fmax = 16;
    F = F < 1 ? 1 : (F > fmax ? fmax : F);
    if (F > 1) F &= ~1;  // even, so that the frame parity is the same in every chunk
    if (F_out) *F_out = F;
    return 2 * static_cast<size_t>(F) * rowbytes + 5 * 33 * sizeof(float);
}
// Largest U+1 the lattice takes: one staged row pair must fit the shared memory of a CTA.
bool lattice_config(int64_t U1, LatCfg *cfg) {
    if (U1 < 1 || U1 > CTCT_MAX_U1 || lattice_smem(U1, nullptr) > kLatticeSmemLimit) return false;
    const int64_t slots = 2 * U1;
    if (slots <= 32) {
        cfg->C = 1;
        cfg->threads = 32;
        return true;
    }
    for (int C = 1; C <= 32; C *= 2) {
        const int per_warp = (C == 1 ? 30 : 31) * C;
        const int64_t warps = (slots + per_warp - 1) / per_warp;
        if (warps <= 32) {
            cfg->C = C;
            cfg->threads = static_cast<int>(warps) * 32;
            return true;
        }
    }
    return false;
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

struct WsLayout {
    size_t G, TAB, LLF, LLI, total;
    LatCfg cfg;
};
bool ws_layout(int64_t N, int64_t T, int64_t U1, int want_grad, WsLayout *w) {
    if (!lattice_config(U1, &w->cfg)) return false;
    const size_t recs = static_cast<size_t>(N) * static_cast<size_t>(T) * static_cast<size_t>(U1);
    size_t o = 0;
    w->G = o;
    o = align256(o + recs * sizeof(float4));
    w->TAB = o;
    if (want_grad) o = align256(o + recs * 2 * sizeof(float4));
    w->LLF = o;
    o = align256(o + static_cast<size_t>(N) * 2 * sizeof(float));
    w->LLI = o;
    o = align256(o + static_cast<size_t>(N) * 2 * sizeof(int));
    w->total = o;
    return true;
}

bool dims_ok(int64_t N, int64_t T, int64_t U1) {
    return N >= 0 && T >= 0 && U1 >= 1 && N <= 65535 && T * U1 < (int64_t(1) << 31) && N * T < (int64_t(1) << 31) &&
           N * T * U1 < (int64_t(1) << 38);
}

const ClearSlice kNoClear = {nullptr, 0, 0, 0};
const PadClear kNoPad = {nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, 1};

// number of clearing blocks a slice adds to a launch
unsigned clear_blocks(const ClearSlice &c) {
    if (!c.ptr) return 0;
    const unsigned long long b = (c.vecs + CLEAR_CHUNK - 1) / CLEAR_CHUNK;
    return static_cast<unsigned>(b ? b : 1);
}

// Split the buffer to clear over the three forward launches (gather, lattice, occupancy gradient).
// Measured at the benchmark shape: clearing beside the gather or the occupancy gradient gains
// nothing (both are bound by the rate of isolated DRAM accesses and slow down by as much as the
// clearing they host), clearing beside the lattice is free (the lattice is bound by its own
// dependent instruction stream).  So the lattice launch takes everything; the split stays
// parametric.  Slices are whole chunks, the last one takes the remainder and the tail.
// all_in_gather: the joint tensor sits in pinned host memory, so the gather launch lasts as long
// as PCIe takes and hides the whole clearing.
void plan_clear(void *clear, size_t bytes, ClearSlice out[3], bool all_in_gather = false) {
    out[0] = out[1] = out[2] = kNoClear;
    if (!clear || !bytes) return;
    const unsigned long long vecs = bytes / 16;
    const unsigned long long chunks = (vecs + CLEAR_CHUNK - 1) / CLEAR_CHUNK;
    const unsigned long long c0 = all_in_gather ? chunks : 0, c2 = 0;
    const unsigned long long c1 = chunks - c0 - c2;
    uint4 *p = static_cast<uint4 *>(clear);
    unsigned long long done = 0;
    const unsigned long long share[3] = {c0, c1, c2};
    for (int i = 0; i < 3; ++i) {
        unsigned long long v = share[i] * CLEAR_CHUNK;
        if (done + v > vecs || i == 2) v = vecs - done;
        if (share[i] == 0 && i != 2) continue;
        out[i].ptr = p + done;
        out[i].vecs = v;
        out[i].tail = 0;
        done += v;
    }
    out[2].tail = static_cast<int>(bytes % 16);
    if (out[2].vecs == 0 && out[2].tail == 0) out[2] = kNoClear;
}

template <int C, int MAXT, int MINB>
int launch_lattice_inst(const LatticeArgs &a, unsigned grid, int block, size_t smem, cudaStream_t st) {
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(k_lattice<C, MAXT, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)) != cudaSuccess)
            return check_launch("lattice smem attribute");
    }
    launch_pdl(k_lattice<C, MAXT, MINB>, dim3(grid), dim3(block), smem, st, a);
    return check_launch("lattice");
}

// `clear`: optional slice that extra blocks of the same launch fill with zeros
int launch_lattice(LatticeArgs a, const LatCfg &cfg, int N, cudaStream_t st, ClearSlice clear = kNoClear,
                   PadClear pad = kNoPad) {
    if (N == 0) return CTCT_OK;
    int F = 1;
    size_t smem = lattice_smem(a.U1, &F);
    a.F = F;
    if (pad.out) clear = kNoClear;  // one kind of clearing per launch
    if ((clear.ptr || pad.out) && smem < CLEAR_TILE_BYTES) smem = CLEAR_TILE_BYTES;  // room for the clearing blocks' zero tile
    if (smem > kLatticeSmemLimit) return CTCT_ERR_UNSUPPORTED;  // lattice_config refuses these sizes up front
    a.smem_bytes = static_cast<unsigned>(smem);
    a.threads = cfg.threads;
    const unsigned own = static_cast<unsigned>(N) * (a.beta_only ? 1 : 2);
    if (pad.out && static_cast<unsigned long long>(pad.slabs) * pad.parts > 0x7ffffff0ull) return CTCT_ERR_UNSUPPORTED;
    const unsigned zero_blocks = pad.out ? pad.slabs * pad.parts : clear_blocks(clear);
    clear.first_block = own;
    a.clear = clear;
    pad.first_block = own;
    a.pad = pad;
    if (static_cast<unsigned long long>(own) + zero_blocks > 0x7fffffffull) return CTCT_ERR_UNSUPPORTED;
    const unsigned grid = own + zero_blocks;
    const int block = (zero_blocks && cfg.threads < 256) ? 256 : cfg.threads;
    // up to 512 threads the kernel is held to 40 registers, so that the clearing blocks of the
    // same launch reach a high occupancy (they need many stores in flight, not registers)
    if (cfg.C == 1 && block <= 512) return launch_lattice_inst<1, 512, 3>(a, grid, block, smem, st);
    switch (cfg.C) {
    case 1: return launch_lattice_inst<1, 1024, 1>(a, grid, block, smem, st);
    case 2: return launch_lattice_inst<2, 1024, 1>(a, grid, block, smem, st);
    case 4: return launch_lattice_inst<4, 1024, 1>(a, grid, block, smem, st);
    case 8: return launch_lattice_inst<8, 1024, 1>(a, grid, block, smem, st);
    case 16: return launch_lattice_inst<16, 1024, 1>(a, grid, block, smem, st);
    case 32: return launch_lattice_inst<32, 1024, 1>(a, grid, block, smem, st);
    }
    return CTCT_ERR_UNSUPPORTED;
}

bool is_pinned_host(const void *p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) == cudaSuccess) return attr.type == cudaMemoryTypeHost;
    cudaGetLastError();
    return false;
}

template <typename InT>
int launch_gather_t(const void *lp, const int *ys, const int *lx, const int *ly, float *out, int64_t N,
                    int64_t T, int64_t U1, int64_t V, bool internal, int valid_only, cudaStream_t st, ClearSlice clear,
                    const int64_t *cu, int64_t packed_rows) {
    const int64_t total = internal ? N * T * U1 * 4 : N * T * U1 * 3;
    if (total == 0) return CTCT_OK;
    // a joint tensor in pinned host memory is read in place: no fill-size hint on those loads
    if (is_pinned_host(lp)) valid_only |= 2;
    // Two independent loads per thread and as many blocks as that takes.  Measured inside the whole step at
    // the benchmark shape (loads per thread / blocks per SM): 4/4 201.8 us per step, 4/8 199.9, 2/16 199.7,
    // 4/unbounded 199.9, 2/unbounded 198.8, 1/unbounded 198.8; the kernel is bound by the rate of isolated
    // DRAM accesses, which more loads in flight per thread do not raise.
    constexpr int kGatherPer = 2;
    const int64_t want = (total + 256 * kGatherPer - 1) / (256 * kGatherPer);
    const int64_t cap = (int64_t(1) << 31) - 1;
    const int own = static_cast<int>(want < cap ? want : cap);
    clear.first_block = static_cast<unsigned>(own);
    const unsigned grid = static_cast<unsigned>(own) + clear_blocks(clear);
    const InT *p = static_cast<const InT *>(lp);
    const bool small = total < (int64_t(1) << 30);  // 32-bit element indices stay clear of overflow in the kernel's strided loop
    if (internal) {
        if (small)
            launch_pdl(k_gather3<InT, unsigned, true, kGatherPer>, dim3(grid), dim3(256), 0, st, p, ys, lx, ly, out, (int)T, (int)U1, (int)V, (unsigned)total, valid_only, clear, cu, packed_rows);
        else
            launch_pdl(k_gather3<InT, unsigned long long, true, kGatherPer>, dim3(grid), dim3(256), 0, st, p, ys, lx, ly, out, (int)T, (int)U1, (int)V, (unsigned long long)total, valid_only, clear, cu, packed_rows);
    } else {
        if (small)
            launch_pdl(k_gather3<InT, unsigned, false, kGatherPer>, dim3(grid), dim3(256), 0, st, p, ys, lx, ly, out, (int)T, (int)U1, (int)V, (unsigned)total, valid_only, clear, cu, packed_rows);
        else
            launch_pdl(k_gather3<InT, unsigned long long, false, kGatherPer>, dim3(grid), dim3(256), 0, st, p, ys, lx, ly, out, (int)T, (int)U1, (int)V, (unsigned long long)total, valid_only, clear, cu, packed_rows);
    }
    return check_launch("gather");
}

int launch_gather(const void *lp, int dtype, const int *ys, const int *lx, const int *ly, float *out, int64_t N,
                  int64_t T, int64_t U1, int64_t V, bool internal, int valid_only, cudaStream_t st,
                  ClearSlice clear = kNoClear, const int64_t *cu = nullptr, int64_t packed_rows = 0) {
    switch (dtype) {
    case CTCT_F32: return launch_gather_t<float>(lp, ys, lx, ly, out, N, T, U1, V, internal, valid_only, st, clear, cu, packed_rows);
    case CTCT_F16: return launch_gather_t<__half>(lp, ys, lx, ly, out, N, T, U1, V, internal, valid_only, st, clear, cu, packed_rows);
    case CTCT_BF16: return launch_gather_t<__nv_bfloat16>(lp, ys, lx, ly, out, N, T, U1, V, internal, valid_only, st, clear, cu, packed_rows);
    }
    return CTCT_ERR_ARG;
}

int launch_fill_grad(const WsLayout &w, char *ws, const int *ys, const int *lx, const int *ly, float *out,
                     int ref_layout, int64_t N, int64_t T, int64_t U1, cudaStream_t st, const float *costs = nullptr,
                     float *loss_out = nullptr, ReduceSpec red = ReduceSpec{0, 0, 1.0f}, ClearSlice clear = kNoClear,
                     int keep_w = 0) {
    if (N == 0) return CTCT_OK;
    if (T == 0) {
        if (loss_out) {
            k_reduce_costs<<<1, 256, 0, st>>>(costs, lx, (int)N, red, loss_out);
            return check_launch("reduce_costs");
        }
        return CTCT_OK;
    }
    GradArgs g;
    g.costs = costs;
    g.loss_out = loss_out;
    g.N = (int)N;
    g.red = red;
    g.G = reinterpret_cast<const float4 *>(ws + w.G);
    g.TAB = reinterpret_cast<const float4 *>(ws + w.TAB);
    g.llf = reinterpret_cast<const float *>(ws + w.LLF);
    g.lli = reinterpret_cast<const int *>(ws + w.LLI);
    g.ys = ys;
    g.lx = lx;
    g.ly = ly;
    g.out = out;
    g.T = (int)T;
    g.U1 = (int)U1;
    g.ref_layout = ref_layout;
    g.keep_w = keep_w;
    g.frames = N * T;
    const unsigned long long own = static_cast<unsigned long long>((g.frames + 7) / 8);  // one warp per frame
    if (own + clear_blocks(clear) > 0x7fffffffull) return CTCT_ERR_UNSUPPORTED;
    clear.first_block = static_cast<unsigned>(own);
    g.clear = clear;
    launch_pdl(k_fill_grad, dim3(static_cast<unsigned>(own) + clear_blocks(clear)), dim3(256), 0, st, g);
    return check_launch("fill_grad");
}

LatticeArgs make_lattice_args(const WsLayout &w, char *ws, const int *ys, const int *lx, const int *ly,
                              float *costs, int64_t T, int64_t U1, int want_grad) {
    LatticeArgs a;
    a.G = reinterpret_cast<const float4 *>(ws + w.G);
    a.ys = ys;
    a.lx = lx;
    a.ly = ly;
    a.TAB = reinterpret_cast<float2 *>(ws + w.TAB);
    a.llf = reinterpret_cast<float *>(ws + w.LLF);
    a.lli = reinterpret_cast<int *>(ws + w.LLI);
    a.costs = costs;
    a.T = (int)T;
    a.U1 = (int)U1;
    a.F = 1;
    a.beta_only = want_grad ? 0 : 1;
    return a;
}

template <typename OutT>
int launch_dense_t(DenseArgs a, int64_t N, cudaStream_t st) {
    const int64_t slabs = N * a.T;
    if (slabs == 0 || a.V == 0) return CTCT_OK;
    constexpr int E = OutOps<OutT>::E;
    a.vec = (a.V % E == 0) && (reinterpret_cast<uintptr_t>(a.out) % 16 == 0);
    k_dense_grad<OutT><<<static_cast<unsigned>(slabs), 256, 0, st>>>(a);
    return check_launch("dense_grad");
}

int launch_logmm(const float *lhs, int64_t lsb, int64_t lsi, int64_t lsk, const float *rhs, int64_t rsb, int64_t rsk,
                 int64_t rsj, int64_t B, int64_t M, int64_t K, int64_t N, float *out, cudaStream_t st,
                 const int *run_flags = nullptr) {
    if (B == 0 || M == 0 || N == 0) return CTCT_OK;
    LogmmArgs a;
    a.lhs = lhs;
    a.rhs = rhs;
    a.out = out;
    a.lsb = lsb;
    a.lsi = lsi;
    a.lsk = lsk;
    a.rsb = rsb;
    a.rsk = rsk;
    a.rsj = rsj;
    a.M = (int)M;
    a.K = (int)K;
    a.N = (int)N;
    a.run_flags = run_flags;
    a.tiles = B * ((M + 31) / 32) * ((N + 31) / 32);
    // stand-by behind the tensor-core kernel (it returns at once unless a flag is up): two blocks per SM,
    // which loop over the tiles if they do have to run; a stand-alone call gets one block per tile
    int64_t blocks = a.tiles;
    if (run_flags && blocks > 2 * static_cast<int64_t>(sm_count())) blocks = 2 * static_cast<int64_t>(sm_count());
    if (blocks > 0x7fffffff) blocks = 0x7fffffff;
    launch_pdl(k_logmm_exact, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, st, a);
    return check_launch("log_matmul");
}

// ---- tensor-core path -----------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// bf16 plane (B, rows, K), K contiguous -> 3-D tensor map with a 64 x 128 x 1 box, 128-byte swizzle
bool make_plane_map(CUtensorMap *map, const void *ptr, int64_t B, int64_t rows, int64_t K, int box_rows = TC_BM) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t gdim[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)B};
    const cuuint64_t gstride[2] = {(cuuint64_t)K * 2, (cuuint64_t)rows * K * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};  // 64 bf16 = one 128-byte swizzle row
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(ptr), gdim, gstride, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// fp32 tensor (B, rows, N), N contiguous -> 3-D tensor map with a 32 x 128 x 1 box, 128-byte swizzle
bool make_f32_tile_map(CUtensorMap *map, const void *ptr, int64_t B, int64_t rows, int64_t N) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t gdim[3] = {(cuuint64_t)N, (cuuint64_t)rows, (cuuint64_t)B};
    const cuuint64_t gstride[2] = {(cuuint64_t)N * 4, (cuuint64_t)rows * N * 4};
    const cuuint32_t box[3] = {32, (cuuint32_t)BW_BM, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(ptr), gdim, gstride, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct TcLayout {
    size_t ah, al, bh, bl, mf, mg, flags, ph, pl, total;
    int64_t Np;  // N rounded up to 8 columns (16-byte rows of the weight planes)
};
TcLayout tc_layout(int64_t B, int64_t M, int64_t N, int64_t K) {
    TcLayout l;
    size_t o = 0;
    l.ah = o; o = align256(o + (size_t)B * M * K * 2);
    l.al = o; o = align256(o + (size_t)B * M * K * 2);
    l.bh = o; o = align256(o + (size_t)B * N * K * 2);
    l.bl = o; o = align256(o + (size_t)B * N * K * 2);
    l.mf = o; o = align256(o + (size_t)B * M * 4);
    l.mg = o; o = align256(o + (size_t)B * N * 4);
    l.flags = o; o = align256(o + 16);
    // backward pass: weight planes P (B, M, Np), bf16 hi and lo
    l.Np = (N + 7) / 8 * 8;
    l.ph = o; o = align256(o + (size_t)B * M * l.Np * 2);
    l.pl = o; o = align256(o + (size_t)B * M * l.Np * 2);
    l.total = o;
    return l;
}
bool tc_shape_ok(int64_t B, int64_t M, int64_t N, int64_t K) {
    return B >= 1 && B <= 65535 && M >= 1 && N >= 1 && K >= 64 && K % 8 == 0 && M < (int64_t(1) << 24) &&
           N <= 65535 * (int64_t)TC_BN && K < (int64_t(1) << 30);
}

template <int VT>
int launch_logmm_bwd_inst(LogmmBwdArgs a, int64_t B, size_t smem, cudaStream_t st) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(k_logmm_bwd_exact<VT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("log_matmul_backward smem attribute");
    a.items = B * ((a.K + VT - 1) / VT);
    // stand-by behind the tensor-core kernels: one block per SM that loops if it does have to run
    int64_t blocks = a.items;
    if (a.run_flags && blocks > static_cast<int64_t>(sm_count())) blocks = sm_count();
    if (blocks > 0x7fffffff) blocks = 0x7fffffff;
    launch_pdl(k_logmm_bwd_exact<VT>, dim3(static_cast<unsigned>(blocks)), dim3(VT), smem, st, a);
    return check_launch("log_matmul_backward");
}

int launch_logmm_bwd(const LogmmBwdArgs &a, int64_t B, cudaStream_t st) {
    if (B == 0 || a.K == 0) return CTCT_OK;
    const size_t limit = 200 * 1024;
    auto need = [&](int vt) { return (2 * static_cast<size_t>(a.Nc) * vt + 2 * static_cast<size_t>(a.Nc)) * sizeof(float); };
    if (need(128) <= limit) return launch_logmm_bwd_inst<128>(a, B, need(128), st);
    if (need(64) <= limit) return launch_logmm_bwd_inst<64>(a, B, need(64), st);
    if (need(32) <= limit) return launch_logmm_bwd_inst<32>(a, B, need(32), st);
    return CTCT_ERR_UNSUPPORTED;
}

template <typename OutT>
int launch_patch_t(const DenseArgs &a, int64_t N, cudaStream_t st) {
    const int64_t rows = N * a.T * a.U1;
    if (rows == 0) return CTCT_OK;
    const int64_t want = (rows + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    const bool sectors = (static_cast<int64_t>(a.V) * sizeof(OutT)) % 32 == 0 && reinterpret_cast<uintptr_t>(a.out) % 32 == 0;
    if (sectors)
        launch_pdl(k_dense_patch<OutT, true>, dim3(static_cast<unsigned>(want < cap ? want : cap)), dim3(256), 0, st, a, rows);
    else
        launch_pdl(k_dense_patch<OutT, false>, dim3(static_cast<unsigned>(want < cap ? want : cap)), dim3(256), 0, st, a, rows);
    return check_launch("dense_patch");
}

template <typename InT>
int launch_lse_gather_t(LseArgs a, cudaStream_t st) {
    a.vec = (a.V % Vec16<InT>::E == 0) && (reinterpret_cast<uintptr_t>(a.logits) % 16 == 0);
    // one block per (n,t) slab; N * T < 2^31 (dims_ok)
    launch_pdl(k_lse_gather<InT>, dim3(static_cast<unsigned>(a.rows / a.U1)), dim3(256), LSE_SMEM_BYTES, st, a);
    return check_launch("lse_gather");
}

int launch_lse_gather(const void *logits, int dtype, const int *ys, const int *lx, const int *ly, float4 *G, int64_t N,
                      int64_t T, int64_t U1, int64_t V, cudaStream_t st, const int64_t *cu, int64_t packed_rows) {
    LseArgs a;
    a.cu = cu;
    a.packed_rows = packed_rows;
    a.logits = logits;
    a.ys = ys;
    a.lx = lx;
    a.ly = ly;
    a.G = G;
    a.T = (int)T;
    a.U1 = (int)U1;
    a.V = (int)V;
    a.rows = N * T * U1;
    a.vec = 0;
    if (a.rows == 0) return CTCT_OK;
    switch (dtype) {
    case CTCT_F32: return launch_lse_gather_t<float>(a, st);
    case CTCT_F16: return launch_lse_gather_t<__half>(a, st);
    case CTCT_BF16: return launch_lse_gather_t<__nv_bfloat16>(a, st);
    }
    return CTCT_ERR_ARG;
}

template <typename T>
int launch_logits_grad_t(LogitsGradArgs a, cudaStream_t st) {
    a.vec = (a.V % Vec16<T>::E == 0) && (reinterpret_cast<uintptr_t>(a.logits) % 16 == 0) &&
            (reinterpret_cast<uintptr_t>(a.out) % 16 == 0);
    launch_pdl(k_logits_grad<T>, dim3(static_cast<unsigned>(a.rows / a.U1)), dim3(256), 0, st, a);
    return check_launch("logits_grad");
}

int dense_backward(DenseArgs a, int64_t N, int dtype, void *stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype != CTCT_F32 && dtype != CTCT_F16 && dtype != CTCT_BF16) return CTCT_ERR_ARG;
    cudaEvent_t *slot = prof_slot(1);
    prof_mark(slot, 0, st);
    int rc = CTCT_ERR_ARG;
    if (a.vec == 2) {  // the buffer was cleared beforehand: only patch
        switch (dtype) {
        case CTCT_F32: rc = launch_patch_t<float>(a, N, st); break;
        case CTCT_F16: rc = launch_patch_t<__half>(a, N, st); break;
        case CTCT_BF16: rc = launch_patch_t<__nv_bfloat16>(a, N, st); break;
        }
    } else {
        switch (dtype) {
        case CTCT_F32: rc = launch_dense_t<float>(a, N, st); break;
        case CTCT_F16: rc = launch_dense_t<__half>(a, N, st); break;
        case CTCT_BF16: rc = launch_dense_t<__nv_bfloat16>(a, N, st); break;
        }
    }
    prof_mark(slot, 1, st);
    return rc;
}

// gather -> lattice -> occupancy gradient (+ optional reduction of the costs into *loss_out)
int forward_impl(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N,
                 int64_t T, int64_t U1, int64_t V, int want_grad, float *costs, float *grads3, void *workspace,
                 size_t workspace_bytes, void *stream, float *loss_out, ReduceSpec red, void *clear = nullptr,
                 size_t clear_bytes = 0, bool from_logits = false, const int64_t *cu = nullptr, int64_t packed_rows = 0) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (dtype != CTCT_F32 && dtype != CTCT_F16 && dtype != CTCT_BF16) return CTCT_ERR_ARG;
    if (N == 0) return CTCT_OK;
    if (!log_probs || !lx || !ly || !costs || (U1 > 1 && !ys) || (want_grad && !grads3)) return CTCT_ERR_ARG;
    WsLayout w;
    if (!ws_layout(N, T, U1, want_grad, &w)) return CTCT_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < w.total || reinterpret_cast<uintptr_t>(workspace) % 256) return CTCT_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);

    if (clear && reinterpret_cast<uintptr_t>(clear) % 16) return CTCT_ERR_ARG;
    ClearSlice cs[3];
    plan_clear((want_grad && !from_logits) ? clear : nullptr, clear_bytes, cs, is_pinned_host(log_probs));
    if (!want_grad && !from_logits && clear && clear_bytes) cs[1] = ClearSlice{static_cast<uint4 *>(clear), clear_bytes / 16, static_cast<int>(clear_bytes % 16), 0};
    cudaEvent_t *slot = prof_slot(from_logits ? 6 : 0);
    prof_mark(slot, 0, st);
    int rc;
    if (from_logits)  // log-softmax fused in: row log-sum-exp and the three picks in one streaming pass
        rc = launch_lse_gather(log_probs, dtype, ys, lx, ly, reinterpret_cast<float4 *>(ws + w.G), N, T, U1, V, st, cu, packed_rows);
    else
        rc = launch_gather(log_probs, dtype, ys, lx, ly, reinterpret_cast<float *>(ws + w.G), N, T, U1, V, true, 1, st, cs[0], cu,
                           packed_rows);
    if (rc) return rc;
    prof_mark(slot, 1, st);
    PadClear pad = kNoPad;
    if (from_logits && clear && want_grad && !cu) {  // `clear` is the gradient buffer of the backward pass: zero its padding rows
        const size_t esize = dtype == CTCT_F32 ? 4 : 2;
        if ((V * esize) % 16 || clear_bytes != static_cast<size_t>(N) * T * U1 * V * esize) return CTCT_ERR_ARG;
        pad.out = static_cast<unsigned char *>(clear);
        pad.lx = lx;
        pad.ly = ly;
        pad.T = (int)T;
        pad.U1 = (int)U1;
        pad.row_bytes = static_cast<unsigned>(V * esize);
        pad.slabs = static_cast<unsigned>(N * T);
        pad.parts = static_cast<unsigned>((static_cast<unsigned long long>(U1) * pad.row_bytes + PAD_PART_BYTES - 1) / PAD_PART_BYTES);
    }
    rc = launch_lattice(make_lattice_args(w, ws, ys, lx, ly, costs, T, U1, want_grad), w.cfg, (int)N, st, cs[1], pad);
    if (rc) return rc;
    prof_mark(slot, 2, st);
    if (want_grad) {
        rc = launch_fill_grad(w, ws, ys, lx, ly, grads3, 0, N, T, U1, st, costs, loss_out, red, cs[2], from_logits ? 1 : 0);
    } else if (loss_out) {
        k_reduce_costs<<<1, 256, 0, st>>>(costs, lx, (int)N, red, loss_out);
        rc = check_launch("reduce_costs");
    }
    prof_mark(slot, 3, st);
    return rc;
}

// Test / benchmark hook: the gather of the forward pass alone (float32 joint tensor, internal record
// layout) with `per` independent loads in flight per thread and a grid of `blocks_per_sm` blocks per SM
// (0: as many blocks as the elements need).
template <int PER>
int gather_probe_t(const float *lp, const int *ys, const int *lx, const int *ly, float *out, int64_t N, int64_t T,
                          int64_t U1, int64_t V, int blocks_per_sm, cudaStream_t st) {
    const int64_t total = N * T * U1 * 4;
    if (total == 0) return CTCT_OK;
    if (total >= (int64_t(1) << 31) - int64_t(1 << 22) * PER) return CTCT_ERR_UNSUPPORTED;
    const int64_t want = (total + 256 * PER - 1) / (256 * PER);
    const int64_t cap = blocks_per_sm > 0 ? static_cast<int64_t>(sm_count()) * blocks_per_sm : want;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    launch_pdl(k_gather3<float, unsigned, true, PER>, dim3(grid), dim3(256), 0, st, lp, ys, lx, ly, out, (int)T, (int)U1, (int)V,
               (unsigned)total, 1, kNoClear, static_cast<const int64_t *>(nullptr), int64_t(0));
    return check_launch("gather_probe");
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
    case CTCT_ERR_STATIC_SCRATCH:
        return "problem needs more scratch than the 32 MiB built into the library; use ctct_b200_loss_forward "
               "with a caller-provided workspace";
    }
    return "unknown error";
}

size_t ctct_b200_grads3_elems(int64_t N, int64_t T, int64_t U1) {
    if (N < 0 || T < 0 || U1 < 1) return 0;
    return static_cast<size_t>(N) * T * U1 * 4;
}

size_t ctct_b200_workspace_bytes(int64_t N, int64_t T, int64_t U1, int want_grad) {
    WsLayout w;
    if (!dims_ok(N, T, U1) || !ws_layout(N, T, U1, want_grad, &w)) return 0;
    return w.total;
}

int ctct_b200_loss_forward(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                           const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int want_grad,
                           float *costs, float *grads3, void *workspace, size_t workspace_bytes, void *stream) {
    return forward_impl(log_probs, dtype, ys, lx, ly, N, T, U1, V, want_grad, costs, grads3, workspace, workspace_bytes,
                        stream, nullptr, ReduceSpec{0, 0, 1.0f});
}

int ctct_b200_loss_forward_reduced(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                                   const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int want_grad,
                                   int reduction, int average_frames, float norm, float *costs, float *loss,
                                   float *grads3, void *workspace, size_t workspace_bytes, void *stream) {
    if ((reduction != 1 && reduction != 2) || !loss || !(norm > 0.0f)) return CTCT_ERR_ARG;
    return forward_impl(log_probs, dtype, ys, lx, ly, N, T, U1, V, want_grad, costs, grads3, workspace, workspace_bytes,
                        stream, loss, ReduceSpec{reduction, average_frames ? 1 : 0, norm});
}

int ctct_b200_loss_forward_fused(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                                 const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int want_grad,
                                 int reduction, int average_frames, float norm, float *costs, float *loss,
                                 float *grads3, void *clear, size_t clear_bytes, void *workspace,
                                 size_t workspace_bytes, void *stream) {
    if (reduction < 0 || reduction > 2) return CTCT_ERR_ARG;
    if (reduction != 0 && (!loss || !(norm > 0.0f))) return CTCT_ERR_ARG;
    return forward_impl(log_probs, dtype, ys, lx, ly, N, T, U1, V, want_grad, costs, grads3, workspace, workspace_bytes,
                        stream, reduction ? loss : nullptr, ReduceSpec{reduction, average_frames ? 1 : 0, reduction ? norm : 1.0f},
                        clear, clear_bytes);
}

int ctct_b200_loss_backward_reduced(const float *grads3, const float *grad_loss, int reduction, int average_frames,
                                    float norm, const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N,
                                    int64_t T, int64_t U1, int64_t V, int dtype, void *dense, void *stream) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if ((reduction != 1 && reduction != 2) || !(norm > 0.0f)) return CTCT_ERR_ARG;
    if (N == 0 || T == 0) return CTCT_OK;
    if (!grads3 || !grad_loss || !lx || !ly || !dense || (U1 > 1 && !ys)) return CTCT_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(grads3) % 16) return CTCT_ERR_ARG;
    DenseArgs a;
    a.GR = reinterpret_cast<const float4 *>(grads3);
    a.grad_out = grad_loss;
    a.ys = ys;
    a.lx = lx;
    a.ly = ly;
    a.out = dense;
    a.T = (int)T;
    a.U1 = (int)U1;
    a.V = (int)V;
    a.vec = 0;
    a.scalar_grad = 1;
    a.red = ReduceSpec{reduction, average_frames ? 1 : 0, norm};
    a.cu = nullptr;
    a.packed_rows = 0;
    return dense_backward(a, N, dtype, stream);
}

int ctct_b200_loss_backward(const float *grads3, const float *grad_out, const int32_t *ys, const int32_t *lx,
                            const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int dtype,
                            void *dense, void *stream) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (N == 0 || T == 0) return CTCT_OK;
    if (!grads3 || !grad_out || !lx || !ly || !dense || (U1 > 1 && !ys)) return CTCT_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(grads3) % 16) return CTCT_ERR_ARG;
    DenseArgs a;
    a.GR = reinterpret_cast<const float4 *>(grads3);
    a.grad_out = grad_out;
    a.ys = ys;
    a.lx = lx;
    a.ly = ly;
    a.out = dense;
    a.T = (int)T;
    a.U1 = (int)U1;
    a.V = (int)V;
    a.vec = 0;
    a.scalar_grad = 0;
    a.red = ReduceSpec{0, 0, 1.0f};
    a.cu = nullptr;
    a.packed_rows = 0;
    return dense_backward(a, N, dtype, stream);
}

int ctct_b200_zero_fill(void *buffer, size_t bytes, void *stream) {
    if (bytes == 0) return CTCT_OK;
    if (!buffer || reinterpret_cast<uintptr_t>(buffer) % 16) return CTCT_ERR_ARG;
    const size_t nvec = bytes / 16;
    const int tail = static_cast<int>(bytes % 16);
    const size_t blocks = (nvec + 1023) / 1024;
    if (blocks > 0x7fffffff) return CTCT_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaEvent_t *slot = prof_slot(2);
    prof_mark(slot, 0, st);
    k_zero_fill<<<static_cast<unsigned>(blocks ? blocks : 1), 256, 0, st>>>(
        static_cast<uint4 *>(buffer), nvec, static_cast<unsigned char *>(buffer) + nvec * 16, tail);
    const int rc = check_launch("zero_fill");
    prof_mark(slot, 1, st);
    return rc;
}

static int backward_patch_impl(const float *grads3, const float *grad, int scalar_grad, int reduction, int average_frames,
                               float norm, const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N, int64_t T,
                               int64_t U1, int64_t V, int dtype, void *dense, void *stream, const int64_t *cu,
                               int64_t packed_rows = 0) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (scalar_grad && ((reduction != 1 && reduction != 2) || !(norm > 0.0f))) return CTCT_ERR_ARG;
    if (N == 0 || T == 0) return CTCT_OK;
    if (!grads3 || !grad || !lx || !ly || !dense || (U1 > 1 && !ys)) return CTCT_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(grads3) % 16) return CTCT_ERR_ARG;
    DenseArgs a;
    a.GR = reinterpret_cast<const float4 *>(grads3);
    a.grad_out = grad;
    a.ys = ys;
    a.lx = lx;
    a.ly = ly;
    a.out = dense;
    a.T = (int)T;
    a.U1 = (int)U1;
    a.V = (int)V;
    a.vec = 2;
    a.scalar_grad = scalar_grad ? 1 : 0;
    a.red = ReduceSpec{scalar_grad ? reduction : 0, average_frames ? 1 : 0, scalar_grad ? norm : 1.0f};
    a.cu = cu;
    a.packed_rows = packed_rows;
    return dense_backward(a, N, dtype, stream);
}

int ctct_b200_loss_backward_patch(const float *grads3, const float *grad, int scalar_grad, int reduction,
                                  int average_frames, float norm, const int32_t *ys, const int32_t *lx,
                                  const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int dtype,
                                  void *dense, void *stream) {
    return backward_patch_impl(grads3, grad, scalar_grad, reduction, average_frames, norm, ys, lx, ly, N, T, U1, V, dtype, dense,
                               stream, nullptr);
}

// ---- packed (ragged) layout: only the valid rows of every utterance exist -----------------------
int ctct_b200_packed_offsets(const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t *cu_rows,
                             void *stream) {
    if (N < 0 || N > 65535 || T < 0 || U1 < 1 || !cu_rows || (N > 0 && (!lx || !ly))) return CTCT_ERR_ARG;
    k_packed_offsets<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(lx, ly, (int)N, (int)T, (int)U1, cu_rows);
    return check_launch("packed_offsets");
}

int ctct_b200_loss_forward_packed(const void *packed, int dtype, const int64_t *cu_rows, int64_t packed_rows, const int32_t *ys,
                                  const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                                  int want_grad, int reduction, int average_frames, float norm, float *costs, float *loss,
                                  float *grads3, void *clear, size_t clear_bytes, void *workspace, size_t workspace_bytes,
                                  void *stream) {
    if (reduction < 0 || reduction > 2 || !cu_rows || packed_rows < 0) return CTCT_ERR_ARG;
    if (reduction != 0 && (!loss || !(norm > 0.0f))) return CTCT_ERR_ARG;
    if (packed && is_pinned_host(packed)) return CTCT_ERR_ARG;
    return forward_impl(packed, dtype, ys, lx, ly, N, T, U1, V, want_grad, costs, grads3, workspace, workspace_bytes, stream,
                        reduction ? loss : nullptr, ReduceSpec{reduction, average_frames ? 1 : 0, reduction ? norm : 1.0f},
                        clear, clear_bytes, false, cu_rows, packed_rows);
}

int ctct_b200_loss_backward_packed(const float *grads3, const float *grad, int scalar_grad, int reduction,
                                   int average_frames, float norm, const int64_t *cu_rows, int64_t packed_rows,
                                   const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N, int64_t T,
                                   int64_t U1, int64_t V, int dtype, void *packed_grad, void *stream) {
    if (!cu_rows || packed_rows < 0) return CTCT_ERR_ARG;
    return backward_patch_impl(grads3, grad, scalar_grad, reduction, average_frames, norm, ys, lx, ly, N, T, U1, V, dtype,
                               packed_grad, stream, cu_rows, packed_rows);
}

int ctct_b200_logits_forward(const void *logits, int dtype, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                             int64_t N, int64_t T, int64_t U1, int64_t V, int want_grad, int reduction,
                             int average_frames, float norm, float *costs, float *loss, float *grads3,
                             void *grad_logits, void *workspace, size_t workspace_bytes, void *stream) {
    if (reduction < 0 || reduction > 2) return CTCT_ERR_ARG;
    if (reduction != 0 && (!loss || !(norm > 0.0f))) return CTCT_ERR_ARG;
    if (logits && is_pinned_host(logits)) return CTCT_ERR_ARG;  // every row is read in full: device memory only
    if (grad_logits && reinterpret_cast<uintptr_t>(grad_logits) % 16) return CTCT_ERR_ARG;
    const size_t esize = dtype == CTCT_F32 ? 4 : 2;
    return forward_impl(logits, dtype, ys, lx, ly, N, T, U1, V, want_grad, costs, grads3, workspace, workspace_bytes, stream,
                        reduction ? loss : nullptr, ReduceSpec{reduction, average_frames ? 1 : 0, reduction ? norm : 1.0f},
                        grad_logits, grad_logits ? static_cast<size_t>(N) * T * U1 * V * esize : 0, true);
}

int ctct_b200_logits_forward_packed(const void *packed_logits, int dtype, const int64_t *cu_rows, int64_t packed_rows,
                                    const int32_t *ys,
                                    const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                                    int want_grad, int reduction, int average_frames, float norm, float *costs, float *loss,
                                    float *grads3, void *workspace, size_t workspace_bytes, void *stream) {
    if (reduction < 0 || reduction > 2 || !cu_rows || packed_rows < 0) return CTCT_ERR_ARG;
    if (reduction != 0 && (!loss || !(norm > 0.0f))) return CTCT_ERR_ARG;
    if (packed_logits && is_pinned_host(packed_logits)) return CTCT_ERR_ARG;
    return forward_impl(packed_logits, dtype, ys, lx, ly, N, T, U1, V, want_grad, costs, grads3, workspace, workspace_bytes,
                        stream, reduction ? loss : nullptr,
                        ReduceSpec{reduction, average_frames ? 1 : 0, reduction ? norm : 1.0f}, nullptr, 0, true, cu_rows,
                        packed_rows);
}

static int logits_backward_impl(const float *grads3, const float *grad, int scalar_grad, int reduction, int average_frames,
                                float norm, const void *logits, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                                int64_t N, int64_t T, int64_t U1, int64_t V, int dtype, void *grad_logits,
                                int padding_cleared, void *stream, const int64_t *cu, int64_t packed_rows = 0) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (dtype != CTCT_F32 && dtype != CTCT_F16 && dtype != CTCT_BF16) return CTCT_ERR_ARG;
    if (scalar_grad && ((reduction != 1 && reduction != 2) || !(norm > 0.0f))) return CTCT_ERR_ARG;
    if (N == 0 || T == 0) return CTCT_OK;
    if (!grads3 || !grad || !logits || !lx || !ly || !grad_logits || (U1 > 1 && !ys)) return CTCT_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(grads3) % 16) return CTCT_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LogitsGradArgs a;
    a.logits = logits;
    a.GR = reinterpret_cast<const float4 *>(grads3);
    a.grad_out = grad;
    a.ys = ys;
    a.lx = lx;
    a.ly = ly;
    a.out = grad_logits;
    a.T = (int)T;
    a.U1 = (int)U1;
    a.V = (int)V;
    a.vec = 0;
    a.scalar_grad = scalar_grad ? 1 : 0;
    a.red = ReduceSpec{scalar_grad ? reduction : 0, average_frames ? 1 : 0, scalar_grad ? norm : 1.0f};
    a.rows = N * T * U1;
    a.padding_cleared = padding_cleared ? 1 : 0;
    a.cu = cu;
    a.packed_rows = packed_rows;
    cudaEvent_t *slot = prof_slot(7);
    prof_mark(slot, 0, st);
    int rc = CTCT_ERR_ARG;
    switch (dtype) {
    case CTCT_F32: rc = launch_logits_grad_t<float>(a, st); break;
    case CTCT_F16: rc = launch_logits_grad_t<__half>(a, st); break;
    case CTCT_BF16: rc = launch_logits_grad_t<__nv_bfloat16>(a, st); break;
    }
    prof_mark(slot, 1, st);
    return rc;
}

int ctct_b200_logits_backward(const float *grads3, const float *grad, int scalar_grad, int reduction, int average_frames,
                              float norm, const void *logits, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                              int64_t N, int64_t T, int64_t U1, int64_t V, int dtype, void *grad_logits,
                              int padding_cleared, void *stream) {
    return logits_backward_impl(grads3, grad, scalar_grad, reduction, average_frames, norm, logits, ys, lx, ly, N, T, U1, V,
                                dtype, grad_logits, padding_cleared, stream, nullptr);
}

int ctct_b200_logits_backward_packed(const float *grads3, const float *grad, int scalar_grad, int reduction,
                                     int average_frames, float norm, const void *packed_logits, const int64_t *cu_rows,
                                     int64_t packed_rows, const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N, int64_t T,
                                     int64_t U1, int64_t V, int dtype, void *packed_grad, void *stream) {
    if (!cu_rows || packed_rows < 0) return CTCT_ERR_ARG;
    return logits_backward_impl(grads3, grad, scalar_grad, reduction, average_frames, norm, packed_logits, ys, lx, ly, N, T, U1,
                                V, dtype, packed_grad, 0, stream, cu_rows, packed_rows);
}

int ctct_b200_gather(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx, const int32_t *ly,
                     int64_t N, int64_t T, int64_t U1, int64_t V, int valid_only, float *gathered, void *stream) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (N == 0 || T == 0) return CTCT_OK;
    if (!log_probs || !gathered || (U1 > 1 && !ys) || (valid_only && (!lx || !ly))) return CTCT_ERR_ARG;
    return launch_gather(log_probs, dtype, ys, lx, ly, gathered, N, T, U1, V, false, valid_only ? 1 : 0,
                         static_cast<cudaStream_t>(stream));
}

int ctct_b200_gather_probe(const float *log_probs, const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N,
                           int64_t T, int64_t U1, int64_t V, int per, int blocks_per_sm, float *records, void *stream) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff || blocks_per_sm < 0 || blocks_per_sm > 32) return CTCT_ERR_ARG;
    if (!log_probs || !lx || !ly || !records || (U1 > 1 && !ys)) return CTCT_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (per) {
    case 1: return gather_probe_t<1>(log_probs, ys, lx, ly, records, N, T, U1, V, blocks_per_sm, st);
    case 2: return gather_probe_t<2>(log_probs, ys, lx, ly, records, N, T, U1, V, blocks_per_sm, st);
    case 4: return gather_probe_t<4>(log_probs, ys, lx, ly, records, N, T, U1, V, blocks_per_sm, st);
    case 8: return gather_probe_t<8>(log_probs, ys, lx, ly, records, N, T, U1, V, blocks_per_sm, st);
    case 16: return gather_probe_t<16>(log_probs, ys, lx, ly, records, N, T, U1, V, blocks_per_sm, st);
    }
    return CTCT_ERR_ARG;
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
    const int64_t total = N * T * U1 * 4;
    if (total > 0) {
        const int64_t want = (total + 255) / 256;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
        k_repack_gathered<<<static_cast<int>(want < cap ? want : cap), 256, 0, st>>>(
            gathered, lx, ly, reinterpret_cast<float *>(ws + w.G), (int)T, (int)U1, total);
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
    e.TAB = reinterpret_cast<const float4 *>(ws + w.TAB);
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
    const int S = 2 * ((int)U1 - 1) + 1;
    const int64_t cells = T * S > 0 ? T * S : 1;
    dim3 grid((unsigned)((cells + 255) / 256), (unsigned)N);
    k_export_tables<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(e);
    return check_launch("export_tables");
}


int ctct_b200_log_matmul(const float *lhs, int64_t lsb, int64_t lsi, int64_t lsk, const float *rhs, int64_t rsb,
                         int64_t rsk, int64_t rsj, int64_t B, int64_t M, int64_t K, int64_t N, float *out,
                         void *stream) {
    if (B < 0 || M < 0 || K < 0 || N < 0 || B > 65535 || M > (int64_t(1) << 20) || N > (int64_t(1) << 20) ||
        K > 0x7fffffff)
        return CTCT_ERR_ARG;
    if (B == 0 || M == 0 || N == 0) return CTCT_OK;
    if (!out || (K > 0 && (!lhs || !rhs))) return CTCT_ERR_ARG;
    return launch_logmm(lhs, lsb, lsi, lsk, rhs, rsb, rsk, rsj, B, M, K, N, out, static_cast<cudaStream_t>(stream));
}


size_t ctct_b200_log_matmul_tc_workspace_bytes(int64_t B, int64_t M, int64_t N, int64_t K) {
    if (!tc_shape_ok(B, M, N, K)) return 0;
    return tc_layout(B, M, N, K).total;
}

int ctct_b200_debug_set_wait_limit(long long polls) {
    const unsigned v = polls < 0 ? TC_SPIN_LIMIT : (polls > 0xffffffffLL ? 0xffffffffu : static_cast<unsigned>(polls));
    if (cudaMemcpyToSymbol(c_tc_spin_limit, &v, sizeof(v)) != cudaSuccess) return check_launch("wait limit");
    return CTCT_OK;
}

size_t ctct_b200_log_matmul_tc_flags_offset(int64_t B, int64_t M, int64_t N, int64_t K) {
    if (!tc_shape_ok(B, M, N, K)) return 0;
    return tc_layout(B, M, N, K).flags;
}

int ctct_b200_log_matmul_tc(const float *f, const float *g, int64_t B, int64_t M, int64_t N, int64_t K, float *den,
                            void *workspace, size_t workspace_bytes, void *stream) {
    if (!tc_shape_ok(B, M, N, K)) return CTCT_ERR_UNSUPPORTED;
    if (!f || !g || !den) return CTCT_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(f) % 16 || reinterpret_cast<uintptr_t>(g) % 16) return CTCT_ERR_ARG;
    const TcLayout l = tc_layout(B, M, N, K);
    if (!workspace || workspace_bytes < l.total || reinterpret_cast<uintptr_t>(workspace) % 256) return CTCT_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);
    auto *ah = reinterpret_cast<__nv_bfloat16 *>(ws + l.ah), *al = reinterpret_cast<__nv_bfloat16 *>(ws + l.al);
    auto *bh = reinterpret_cast<__nv_bfloat16 *>(ws + l.bh), *bl = reinterpret_cast<__nv_bfloat16 *>(ws + l.bl);
    float *mf = reinterpret_cast<float *>(ws + l.mf), *mg = reinterpret_cast<float *>(ws + l.mg);
    int *flags = reinterpret_cast<int *>(ws + l.flags);
    CUtensorMap m_ah, m_al, m_bh, m_bl;
    if (!make_plane_map(&m_ah, ah, B, M, K) || !make_plane_map(&m_al, al, B, M, K) ||
        !make_plane_map(&m_bh, bh, B, N, K) || !make_plane_map(&m_bl, bl, B, N, K)) {
        snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "cuTensorMapEncodeTiled failed");
        return CTCT_ERR_LAUNCH;
    }
    if (cudaMemsetAsync(flags, 0, 16, st) != cudaSuccess) return check_launch("log_matmul_tc flags");
    cudaEvent_t *slot = prof_slot(3);
    prof_mark(slot, 0, st);
    launch_pdl(k_exp_split, dim3(static_cast<unsigned>(B * M)), dim3(256), 0, st, f, (int)K, ah, al, mf);
    int rc = check_launch("exp_split f");
    if (rc) return rc;
    launch_pdl(k_exp_split, dim3(static_cast<unsigned>(B * N)), dim3(256), 0, st, g, (int)K, bh, bl, mg);
    rc = check_launch("exp_split g");
    if (rc) return rc;
    prof_mark(slot, 1, st);
    // the attribute belongs to the current device, so it is set on every launch (as for the lattice)
    if (cudaFuncSetAttribute(k_logmm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES) != cudaSuccess)
        return check_launch("log_matmul_tc smem attribute");
    LogmmTcArgs a;
    a.den = den;
    a.mf = mf;
    a.mg = mg;
    a.M = (int)M;
    a.N = (int)N;
    a.K = (int)K;
    a.flags = flags;
    dim3 grid((unsigned)((M + TC_BM - 1) / TC_BM), (unsigned)((N + TC_BN - 1) / TC_BN), (unsigned)B);
    launch_pdl(k_logmm_tc, grid, dim3(128), TC_SMEM_BYTES, st, m_ah, m_al, m_bh, m_bl, a);
    rc = check_launch("log_matmul_tc");
    if (rc) return rc;
    prof_mark(slot, 2, st);
    // exact kernel, a no-op unless a wait ran out or a shifted sum underflowed
    rc = launch_logmm(f, M * K, K, 1, g, N * K, 1, K, B, M, K, N, den, st, flags);
    prof_mark(slot, 3, st);
    return rc;
}

int ctct_b200_log_matmul_backward(const float *grad_out, const float *lhs, const float *rhsT, const float *res,
                                  int64_t B, int64_t M, int64_t K, int64_t N, float *grad_lhs, float *grad_rhsT,
                                  void *stream) {
    if (B < 0 || M < 0 || K < 0 || N < 0 || B > 65535 || K > 0x7fffffff || M > 0x7fffffff || N > 0x7fffffff)
        return CTCT_ERR_ARG;
    if (B == 0 || K == 0) return CTCT_OK;
    if (!grad_out || !lhs || !rhsT || !res) return CTCT_ERR_ARG;
    LogmmBwdArgs a = {};
    a.lhs = lhs;
    a.rhsT = rhsT;
    a.res = res;
    a.gout = grad_out;
    a.grad_lhs = grad_lhs;
    a.grad_rhsT = grad_rhsT;
    a.M = (int)M;
    a.Nc = (int)N;
    a.K = (int)K;
    return launch_logmm_bwd(a, B, static_cast<cudaStream_t>(stream));
}

int ctct_b200_simple_forward(const float *f, const float *g, const float *den, const int32_t *ys, const int32_t *lx,
                             const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V, int want_grad,
                             float *costs, float *grads3, void *workspace, size_t workspace_bytes, void *stream) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (N == 0) return CTCT_OK;
    if (!f || !g || !lx || !ly || !costs || (U1 > 1 && !ys) || (want_grad && !grads3)) return CTCT_ERR_ARG;
    WsLayout w;
    if (!ws_layout(N, T, U1, want_grad, &w)) return CTCT_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < w.total || reinterpret_cast<uintptr_t>(workspace) % 256) return CTCT_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);
    ComposeArgs c;
    c.f = f;
    c.g = g;
    c.den = den;
    c.ys = ys;
    c.lx = lx;
    c.ly = ly;
    c.G = reinterpret_cast<float *>(ws + w.G);
    c.T = (int)T;
    c.U1 = (int)U1;
    c.V = (int)V;
    c.total = N * T * U1 * 4;
    cudaEvent_t *slot = prof_slot(4);
    prof_mark(slot, 0, st);
    if (c.total > 0) {
        const dim3 grid(static_cast<unsigned>((T + COMPOSE_FRAMES - 1) / COMPOSE_FRAMES), static_cast<unsigned>(N));
        const size_t smem = static_cast<size_t>(U1) * 3 * sizeof(float);
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(k_simple_compose, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
            return check_launch("simple_compose smem attribute");
        launch_pdl(k_simple_compose, grid, dim3(256), smem, st, c);
        int rc = check_launch("simple_compose");
        if (rc) return rc;
    }
    prof_mark(slot, 1, st);
    int rc = launch_lattice(make_lattice_args(w, ws, ys, lx, ly, costs, T, U1, want_grad), w.cfg, (int)N, st);
    if (rc) return rc;
    prof_mark(slot, 2, st);
    if (want_grad) rc = launch_fill_grad(w, ws, ys, lx, ly, grads3, 0, N, T, U1, st);
    prof_mark(slot, 3, st);
    return rc;
}

size_t ctct_b200_simple_gathered_workspace_bytes(int64_t N, int64_t T, int64_t U1, int want_grad) {
    WsLayout w;
    if (!dims_ok(N, T, U1) || !ws_layout(N, T, U1, want_grad, &w)) return 0;
    return w.total + (want_grad ? align256(static_cast<size_t>(N) * T * U1 * sizeof(float4)) : 0);
}

int ctct_b200_simple_gathered_forward(const float *f, const float *g, const float *den, const int32_t *ys,
                                      const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1,
                                      int want_grad, float *costs, float *grad_f, float *grad_g, float *grad_den,
                                      void *workspace, size_t workspace_bytes, void *stream) {
    if (!dims_ok(N, T, U1)) return CTCT_ERR_ARG;
    if (N == 0) return CTCT_OK;
    if (!f || !g || !lx || !ly || !costs || (U1 > 1 && !ys)) return CTCT_ERR_ARG;
    if (want_grad && (!grad_f || !grad_g || (den && !grad_den))) return CTCT_ERR_ARG;
    WsLayout w;
    if (!ws_layout(N, T, U1, want_grad, &w)) return CTCT_ERR_UNSUPPORTED;
    const size_t need = w.total + (want_grad ? align256(static_cast<size_t>(N) * T * U1 * sizeof(float4)) : 0);
    if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256) return CTCT_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char *ws = static_cast<char *>(workspace);
    float *grads3 = reinterpret_cast<float *>(ws + w.total);
    GatheredArgs c;
    c.f = f;
    c.g = g;
    c.den = den;
    c.lx = lx;
    c.ly = ly;
    c.G = reinterpret_cast<float4 *>(ws + w.G);
    c.T = (int)T;
    c.U1 = (int)U1;
    c.rows = N * T * U1;
    if (c.rows > 0) {
        const int64_t want = (c.rows + 255) / 256;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
        launch_pdl(k_gathered_compose, dim3(static_cast<unsigned>(want < cap ? want : cap)), dim3(256), 0, st, c);
        int rc = check_launch("gathered_compose");
        if (rc) return rc;
    }
    int rc = launch_lattice(make_lattice_args(w, ws, ys, lx, ly, costs, T, U1, want_grad), w.cfg, (int)N, st);
    if (rc || !want_grad) return rc;
    rc = launch_fill_grad(w, ws, ys, lx, ly, grads3, 0, N, T, U1, st);
    if (rc || T == 0) return rc;
    GatheredReduceArgs r;
    r.grads3 = reinterpret_cast<const float4 *>(grads3);
    r.lx = lx;
    r.ly = ly;
    r.grad_f = grad_f;
    r.grad_g = grad_g;
    r.grad_den = den ? grad_den : nullptr;
    r.N = (int)N;
    r.T = (int)T;
    r.U1 = (int)U1;
    launch_pdl(k_gathered_reduce_t, dim3(static_cast<unsigned>((N * T + 7) / 8)), dim3(256), 0, st, r);
    rc = check_launch("gathered_reduce_t");
    if (rc) return rc;
    launch_pdl(k_gathered_reduce_u, dim3(static_cast<unsigned>((N * U1 + 7) / 8)), dim3(256), 0, st, r);
    return check_launch("gathered_reduce_u");
}

// tensor-core gradient through the denominator; planes, maxima and flags are those the forward
// pass (ctct_b200_log_matmul_tc) left in tc_ws
// grad_f: short contraction (U+1), the output stream dominates -> three epilogue tiles in flight;
// grad_g: long contraction (T) over the big Ef planes -> deep operand ring
constexpr int BW_F_STAGES = 2, BW_F_EBUFS = 3, BW_G_STAGES = 4, BW_G_EBUFS = 1;
// grad_f with U+1 <= 128: the weight tile stays in shared memory (64 KB), only Eg streams (16 KB stages)
constexpr int BW_R_STAGES = 4, BW_R_EBUFS = 3;
static int den_backward_tc(const float4 *g4, const float *gout, const float *grad_out, const float *f, const float *g, const float *den,
                           const int32_t *lx, const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                           float *grad_f, float *grad_g, char *ws, const TcLayout &l, cudaEvent_t *slot,
                           cudaStream_t st) {
    auto *ah = reinterpret_cast<__nv_bfloat16 *>(ws + l.ah), *al = reinterpret_cast<__nv_bfloat16 *>(ws + l.al);
    auto *bh = reinterpret_cast<__nv_bfloat16 *>(ws + l.bh), *bl = reinterpret_cast<__nv_bfloat16 *>(ws + l.bl);
    auto *ph = reinterpret_cast<__nv_bfloat16 *>(ws + l.ph), *pl = reinterpret_cast<__nv_bfloat16 *>(ws + l.pl);
    float *mf = reinterpret_cast<float *>(ws + l.mf), *mg = reinterpret_cast<float *>(ws + l.mg);
    int *flags = reinterpret_cast<int *>(ws + l.flags);
    DenWeightArgs w;
    w.grads3 = g4;
    w.scale = grad_out;
    w.gout = gout;
    w.den = den;
    w.mf = mf;
    w.mg = mg;
    w.lx = lx;
    w.ly = ly;
    w.ph = ph;
    w.pl = pl;
    w.T = (int)T;
    w.U1 = (int)U1;
    w.U1p = (int)l.Np;
    w.flags = flags;
    launch_pdl(k_den_weights, dim3(static_cast<unsigned>(N * T)), dim3(128), 0, st, w);
    int rc = check_launch("den_weights");
    if (rc) return rc;
    CUtensorMap m_pk_h, m_pk_l, m_pm_h, m_pm_l, m_f_h, m_f_l, m_g_h, m_g_l;
    if (!make_plane_map(&m_pk_h, ph, N, T, l.Np, BW_BM) || !make_plane_map(&m_pk_l, pl, N, T, l.Np, BW_BM) ||
        !make_plane_map(&m_pm_h, ph, N, T, l.Np, BW_BK) || !make_plane_map(&m_pm_l, pl, N, T, l.Np, BW_BK) ||
        !make_plane_map(&m_f_h, ah, N, T, V, BW_BK) || !make_plane_map(&m_f_l, al, N, T, V, BW_BK) ||
        !make_plane_map(&m_g_h, bh, N, U1, V, BW_BK) || !make_plane_map(&m_g_l, bl, N, U1, V, BW_BK)) {
        snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "cuTensorMapEncodeTiled failed");
        return CTCT_ERR_LAUNCH;
    }
    if (grad_f && grad_g && U1 <= 128) {
        // both gradients in one pass over the Ef planes (shared-memory attribute: per device, so per launch)
        if (cudaFuncSetAttribute(k_den_bwd_fused, cudaFuncAttributeMaxDynamicSharedMemorySize, FU_SMEM_BYTES) != cudaSuccess)
            return check_launch("den_bwd_fused smem attribute");
        CUtensorMap m_out;
        if (!make_f32_tile_map(&m_out, grad_f, N, T, V)) {
            snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "cuTensorMapEncodeTiled failed");
            return CTCT_ERR_LAUNCH;
        }
        DenBwdFusedArgs fa;
        fa.g = g;
        fa.mg = mg;
        fa.grad_g = grad_g;
        fa.T = (int)T;
        fa.U1 = (int)U1;
        fa.V = (int)V;
        fa.slabs = (int)((V + FU_V - 1) / FU_V);
        const int64_t items = (int64_t)fa.slabs * N;
        if (items > 0x7fffffff) return CTCT_ERR_UNSUPPORTED;
        fa.items = (int)items;
        fa.flags = flags;
        const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());
        launch_pdl(k_den_bwd_fused, dim3(grid), dim3(FU_THREADS), FU_SMEM_BYTES, st, m_pk_h, m_pk_l, m_f_h, m_f_l, m_g_h,
                   m_g_l, m_out, fa);
        rc = check_launch("den_bwd_fused");
        prof_mark(slot, 1, st);
        return rc;
    }
    const int tiles_n = (int)((V + BW_BN - 1) / BW_BN);
    auto launch = [&](bool a_mn, const CUtensorMap &pa_h, const CUtensorMap &pa_l, const CUtensorMap &pb_h,
                      const CUtensorMap &pb_l, const float *src, const float *mx, float *out, int64_t M, int64_t K,
                      const char *what) -> int {
        CUtensorMap m_src, m_out;
        if (!make_f32_tile_map(&m_src, src, N, M, V) || !make_f32_tile_map(&m_out, out, N, M, V)) {
            snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "cuTensorMapEncodeTiled failed");
            return CTCT_ERR_LAUNCH;
        }
        LogmmBwdTcArgs a;
        a.mx = mx;
        a.M = (int)M;
        a.N = (int)V;
        a.K = (int)K;
        a.tiles_m = (int)((M + BW_BM - 1) / BW_BM);
        a.tiles_n = tiles_n;
        const int64_t total = (int64_t)a.tiles_m * tiles_n * N;
        if (total > 0x7fffffff) return CTCT_ERR_UNSUPPORTED;
        a.total_tiles = (int)total;
        a.flags = flags;
        const unsigned grid = (unsigned)(total < sm_count() ? total : sm_count());
        // shared-memory attributes belong to the current device: set with every launch
        auto smem_attr = [](auto kernel, int bytes) {
            return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
        };
        const bool attr_ok =
            a_mn ? smem_attr(k_logmm_bwd_tc<true, false, BW_G_STAGES, BW_G_EBUFS>, bw_smem_bytes(BW_G_STAGES, BW_G_EBUFS, false))
            : (K <= BW_BK * BW_ARES_KB)
                ? smem_attr(k_logmm_bwd_tc<false, true, BW_R_STAGES, BW_R_EBUFS>, bw_smem_bytes(BW_R_STAGES, BW_R_EBUFS, true))
                : smem_attr(k_logmm_bwd_tc<false, false, BW_F_STAGES, BW_F_EBUFS>, bw_smem_bytes(BW_F_STAGES, BW_F_EBUFS, false));
        if (!attr_ok) return check_launch("logmm_bwd_tc smem attribute");
        if (a_mn)
            launch_pdl(k_logmm_bwd_tc<true, false, BW_G_STAGES, BW_G_EBUFS>, dim3(grid), dim3(BW_THREADS),
                       bw_smem_bytes(BW_G_STAGES, BW_G_EBUFS, false), st, pa_h, pa_l, pb_h, pb_l, m_src, m_out, a);
        else if (K <= BW_BK * BW_ARES_KB)  // the whole contraction of A fits the resident buffer
            launch_pdl(k_logmm_bwd_tc<false, true, BW_R_STAGES, BW_R_EBUFS>, dim3(grid), dim3(BW_THREADS),
                       bw_smem_bytes(BW_R_STAGES, BW_R_EBUFS, true), st, pa_h, pa_l, pb_h, pb_l, m_src, m_out, a);
        else
            launch_pdl(k_logmm_bwd_tc<false, false, BW_F_STAGES, BW_F_EBUFS>, dim3(grid), dim3(BW_THREADS),
                       bw_smem_bytes(BW_F_STAGES, BW_F_EBUFS, false), st, pa_h, pa_l, pb_h, pb_l, m_src, m_out, a);
        return check_launch(what);
    };
    // grad_f[t,v] = Ef[t,v] * sum_u P[t,u] Eg[u,v]
    if (grad_f && (rc = launch(false, m_pk_h, m_pk_l, m_g_h, m_g_l, f, mf, grad_f, T, U1, "logmm_bwd_tc grad_f"))) return rc;
    prof_mark(slot, 1, st);
    // grad_g[u,v] = Eg[u,v] * sum_t P[t,u] Ef[t,v]
    if (grad_g && (rc = launch(true, m_pm_h, m_pm_l, m_f_h, m_f_l, g, mg, grad_g, U1, T, "logmm_bwd_tc grad_g"))) return rc;
    return CTCT_OK;
}

static int simple_backward_impl(const float *grads3, const float *grad_out, const float *f, const float *g,
                                const float *den, const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N,
                                int64_t T, int64_t U1, int64_t V, float *grad_f, float *grad_g, void *tc_ws,
                                size_t tc_ws_bytes, void *stream) {
    if (!dims_ok(N, T, U1) || V < 1 || V > 0x7fffffff) return CTCT_ERR_ARG;
    if (N == 0) return CTCT_OK;
    if (!grads3 || !grad_out || !lx || !ly || (U1 > 1 && !ys) || (den && (!f || !g))) return CTCT_ERR_ARG;
    if (!grad_f && !grad_g) return CTCT_OK;
    if (reinterpret_cast<uintptr_t>(grads3) % 16) return CTCT_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const float4 *g4 = reinterpret_cast<const float4 *>(grads3);
    cudaEvent_t *slot = prof_slot(5);
    prof_mark(slot, 0, st);
    if (den) {
        const int *run_flags = nullptr;
        if (tc_ws) {
            if (!tc_shape_ok(N, T, U1, V)) return CTCT_ERR_UNSUPPORTED;
            const TcLayout l = tc_layout(N, T, U1, V);
            if (tc_ws_bytes < l.total || reinterpret_cast<uintptr_t>(tc_ws) % 256) return CTCT_ERR_WORKSPACE;
            if (reinterpret_cast<uintptr_t>(f) % 16 || reinterpret_cast<uintptr_t>(g) % 16 ||
                (grad_f && reinterpret_cast<uintptr_t>(grad_f) % 16) || (grad_g && reinterpret_cast<uintptr_t>(grad_g) % 16))
                return CTCT_ERR_ARG;
            int rc = den_backward_tc(g4, nullptr, grad_out, f, g, den, lx, ly, N, T, U1, V, grad_f, grad_g,
                                     static_cast<char *>(tc_ws), l, slot, st);
            if (rc) return rc;
            run_flags = reinterpret_cast<const int *>(static_cast<char *>(tc_ws) + l.flags);
        }
        // exact kernel: the whole job without a tensor-core workspace, otherwise a no-op unless a
        // flag in that workspace says the tensor-core result cannot be used
        LogmmBwdArgs a = {};
        a.lhs = f;
        a.rhsT = g;
        a.res = den;
        a.grads3 = g4;
        a.scale = grad_out;
        a.lx = lx;
        a.ly = ly;
        a.grad_lhs = grad_f;
        a.grad_rhsT = grad_g;
        a.M = (int)T;
        a.Nc = (int)U1;
        a.K = (int)V;
        a.run_flags = run_flags;
        int rc = launch_logmm_bwd(a, N, st);
        if (rc) return rc;
    } else {
        if (grad_f && cudaMemsetAsync(grad_f, 0, sizeof(float) * N * T * V, st) != cudaSuccess) return check_launch("memset grad_f");
        if (grad_g && cudaMemsetAsync(grad_g, 0, sizeof(float) * N * U1 * V, st) != cudaSuccess) return check_launch("memset grad_g");
    }
    if (!(den && tc_ws)) prof_mark(slot, 1, st);  // without the tensor-core path the second interval is empty
    prof_mark(slot, 2, st);
    PatchArgs p;
    p.grads3 = g4;
    p.scale = grad_out;
    p.ys = ys;
    p.lx = lx;
    p.ly = ly;
    p.grad_f = grad_f;
    p.grad_g = grad_g;
    p.T = (int)T;
    p.U1 = (int)U1;
    p.V = (int)V;
    if (grad_f && grad_g && T > 0) {  // both: one launch, side by side
        const int g_blocks = (int)((U1 + 31) / 32);
        dim3 grid((unsigned)(g_blocks + (T + 7) / 8), (unsigned)N);
        launch_pdl(k_simple_patch_fg, grid, dim3(256), 0, st, p, g_blocks);
        int rc = check_launch("simple_patch_fg");
        if (rc) return rc;
        prof_mark(slot, 3, st);
        return CTCT_OK;
    }
    if (grad_f && T > 0) {
        dim3 grid((unsigned)((T + 7) / 8), (unsigned)N);  // one warp per frame
        launch_pdl(k_simple_patch_f, grid, dim3(256), 0, st, p);
        int rc = check_launch("simple_patch_f");
        if (rc) return rc;
    }
    if (grad_g) {
        launch_pdl(k_simple_patch_g, dim3((unsigned)((U1 + 31) / 32), (unsigned)N), dim3(256), 0, st, p, (int)N);
        int rc = check_launch("simple_patch_g");
        if (rc) return rc;
    }
    prof_mark(slot, 3, st);
    return CTCT_OK;
}

int ctct_b200_log_matmul_backward_tc(const float *grad_out, const float *lhs, const float *rhsT, const float *res,
                                     int64_t B, int64_t M, int64_t K, int64_t N, float *grad_lhs, float *grad_rhsT,
                                     void *tc_workspace, size_t tc_workspace_bytes, void *stream) {
    if (!tc_shape_ok(B, M, N, K)) return CTCT_ERR_UNSUPPORTED;
    if (!grad_out || !lhs || !rhsT || !res || !tc_workspace) return CTCT_ERR_ARG;
    if (!grad_lhs && !grad_rhsT) return CTCT_OK;
    const TcLayout l = tc_layout(B, M, N, K);
    if (tc_workspace_bytes < l.total || reinterpret_cast<uintptr_t>(tc_workspace) % 256) return CTCT_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = den_backward_tc(nullptr, grad_out, nullptr, lhs, rhsT, res, nullptr, nullptr, B, M, N, K, grad_lhs, grad_rhsT,
                             static_cast<char *>(tc_workspace), l, nullptr, st);
    if (rc) return rc;
    // exact kernel: a no-op unless a flag in the workspace says the tensor-core result cannot be used
    LogmmBwdArgs a = {};
    a.lhs = lhs;
    a.rhsT = rhsT;
    a.res = res;
    a.gout = grad_out;
    a.grad_lhs = grad_lhs;
    a.grad_rhsT = grad_rhsT;
    a.M = (int)M;
    a.Nc = (int)N;
    a.K = (int)K;
    a.run_flags = reinterpret_cast<const int *>(static_cast<char *>(tc_workspace) + l.flags);
    return launch_logmm_bwd(a, B, st);
}

int ctct_b200_simple_backward(const float *grads3, const float *grad_out, const float *f, const float *g,
                              const float *den, const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N,
                              int64_t T, int64_t U1, int64_t V, float *grad_f, float *grad_g, void *stream) {
    return simple_backward_impl(grads3, grad_out, f, g, den, ys, lx, ly, N, T, U1, V, grad_f, grad_g, nullptr, 0, stream);
}

int ctct_b200_simple_backward_tc(const float *grads3, const float *grad_out, const float *f, const float *g,
                                 const float *den, const int32_t *ys, const int32_t *lx, const int32_t *ly, int64_t N,
                                 int64_t T, int64_t U1, int64_t V, float *grad_f, float *grad_g, void *tc_workspace,
                                 size_t tc_workspace_bytes, void *stream) {
    if (!tc_workspace || !den) return CTCT_ERR_ARG;
    return simple_backward_impl(grads3, grad_out, f, g, den, ys, lx, ly, N, T, U1, V, grad_f, grad_g, tc_workspace,
                                tc_workspace_bytes, stream);
}

static int profile_disable_locked() {
    if (g_prof.ev) {
        for (int i = 0; i < 4 * g_prof.cap; ++i) cudaEventDestroy(g_prof.ev[i]);
        delete[] g_prof.ev;
        delete[] g_prof.kind;
    }
    g_prof = Profiler();
    return CTCT_OK;
}

int ctct_b200_profile_disable(void) {
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    return profile_disable_locked();
}

int ctct_b200_profile_enable(int max_calls) {
    if (max_calls < 1 || max_calls > (1 << 20)) return CTCT_ERR_ARG;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    profile_disable_locked();
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
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    const int n = g_prof.used < capacity ? g_prof.used : capacity;
    for (int i = 0; i < n; ++i) {
        cudaEvent_t *e = g_prof.ev + 4 * i;
        const int k_ = g_prof.kind[i];
        const int pairs = (k_ == 0 || (k_ >= 3 && k_ <= 6)) ? 3 : 1;  // intervals recorded per kind
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

// ---------------------------------------------------------------------------------------
// Forward without a caller-provided workspace: the scratch is a fixed array in the device image.
// In host code `g_noalloc_scratch` is only a handle for the symbol, never a device address; the
// address the kernels get comes from cudaGetSymbolAddress, looked up once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CTCT_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void *g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;
}  // namespace

extern "C" int ctct_b200_loss_forward_noalloc(const void *log_probs, int dtype, const int32_t *ys, const int32_t *lx,
                                              const int32_t *ly, int64_t N, int64_t T, int64_t U1, int64_t V,
                                              int want_grad, float *costs, float *grads3, void *stream) {
    if (!dims_ok(N, T, U1)) return CTCT_ERR_ARG;
    if (N == 0) return CTCT_OK;
    WsLayout w;
    if (!ws_layout(N, T, U1, want_grad, &w)) return CTCT_ERR_UNSUPPORTED;
    if (w.total > CTCT_NOALLOC_SCRATCH_BYTES) return CTCT_ERR_STATIC_SCRATCH;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        if (check_launch("noalloc device") == CTCT_OK) snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "noalloc: no current device");
        return CTCT_ERR_LAUNCH;
    }
    if (dev < 0 || dev >= kMaxDevices) return CTCT_ERR_UNSUPPORTED;  // device ordinal beyond the address cache
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_ptr[dev]) {
            void *p = nullptr;
            if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) {
                // never report success with nothing launched
                if (check_launch("noalloc symbol address") == CTCT_OK)
                    snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "noalloc: cudaGetSymbolAddress returned no address");
                return CTCT_ERR_LAUNCH;
            }
            g_noalloc_ptr[dev] = p;
        }
        scratch = g_noalloc_ptr[dev];
    }
    return ctct_b200_loss_forward(log_probs, dtype, ys, lx, ly, N, T, U1, V, want_grad, costs, grads3, scratch,
                                  CTCT_NOALLOC_SCRATCH_BYTES, stream);
}
