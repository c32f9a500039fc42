"""The allocation-free forward entry point, ctct_b200_loss_forward_noalloc.

Some users of the library may not allocate device memory when they call it (a plug-in whose host
application owns all GPU memory, a real-time loop that cannot afford the synchronisation an
allocation implies).  For them the library carries a fixed 32 MiB scratch array in its device
image.  This file checks, through the C ABI, that the entry point gives the same costs and
compact gradient as ctct_b200_loss_forward with a caller-provided workspace, on two calls in a
row (the second call finds the first call's leftovers in the shared array), that both agree with
the CPU oracle, and that a problem too large for the array is refused.  It is named so that
pytest collects it last.
"""
import numpy as np
import pytest
import torch

import oracle
from util import make_case

DEV = "cuda:0"


def _forward(lib, name, lp_t, ys_t, lx_t, ly_t, with_workspace):
    from warp_ctct_b200 import _lib
    N, T, U1, V = lp_t.shape
    dev = torch.device(DEV)
    costs = torch.full((N,), float("nan"), device=dev)
    grads3 = torch.full((lib.ctct_b200_grads3_elems(N, T, U1),), float("nan"), device=dev)
    args = [lp_t.data_ptr(), _lib.dtype_code(lp_t.dtype), ys_t.data_ptr(), lx_t.data_ptr(), ly_t.data_ptr(),
            N, T, U1, V, 1, costs.data_ptr(), grads3.data_ptr()]
    if with_workspace:
        ws = _lib.workspace(N, T, U1, True, dev)
        rc = lib.ctct_b200_loss_forward(*args, ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev))
    else:
        rc = lib.ctct_b200_loss_forward_noalloc(*args, _lib.stream_ptr(dev))
    _lib.check(rc, name)
    torch.cuda.synchronize()
    return costs.cpu().numpy(), grads3.view(N, T, U1, 4).cpu().numpy()


@pytest.mark.gpu
def test_noalloc_forward_matches_workspace_forward_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from warp_ctct_b200 import _lib
    lib = _lib.lib()
    # two different problems back to back: the second runs over the first one's scratch contents
    cases = [make_case(6, 40, 17, 64, 1.5, 301, lx_range=(20, 40), ly_range=(2, 16), repeat_prob=0.2),
             make_case(3, 70, 40, 33, 1.5, 302, lx_range=(50, 70), ly_range=(10, 39))]
    for lp, ys, lx, ly in cases:
        lp_t, ys_t, lx_t, ly_t = [torch.from_numpy(np.ascontiguousarray(a)).to(DEV) for a in (lp, ys, lx, ly)]
        c_ref, g_ref = _forward(lib, "loss_forward", lp_t, ys_t, lx_t, ly_t, with_workspace=True)
        # the CPU oracle on the same inputs (float64 evaluation of the reference's formulas)
        c64, g64 = oracle.ctct_fwd(oracle.collect_units(lp, ys), ys, lx, ly, True, np.float64)
        for attempt in range(2):
            c, g = _forward(lib, "loss_forward_noalloc", lp_t, ys_t, lx_t, ly_t, with_workspace=False)
            assert np.isfinite(c_ref).all()
            np.testing.assert_allclose(c, c_ref, rtol=1e-5, err_msg=f"call {attempt}")
            assert np.abs(g - g_ref).max() < 1e-4, attempt
            np.testing.assert_allclose(c, c64, rtol=1e-5, err_msg=f"call {attempt} against the oracle")
            assert np.abs(g[..., :3] - g64).max() < 1e-4, attempt
            assert not g[..., 3].any()
    # a problem whose workspace exceeds the built-in array is refused before any launch
    N, T, U1, V = 64, 400, 101, 8
    assert lib.ctct_b200_workspace_bytes(N, T, U1, 1) > 32 << 20
    x = torch.zeros(8, device=DEV)
    rc = lib.ctct_b200_loss_forward_noalloc(x.data_ptr(), 0, x.data_ptr(), x.data_ptr(), x.data_ptr(), N, T, U1, V, 1,
                                            x.data_ptr(), x.data_ptr(), None)
    assert rc == -5
    with pytest.raises(RuntimeError, match="32 MiB"):
        _lib.check(rc, "loss_forward_noalloc")
