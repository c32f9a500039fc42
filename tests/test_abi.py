"""CPU checks of the drop-in boundary: the shared library loads, exports exactly what the header
declares, and the Python surface mirrors the reference's signatures.  No kernel is launched."""
import ctypes
import inspect
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "ctct_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ctct_b200_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def built():
    from warp_ctct_b200 import build
    return build.build()


def test_header_declares_entry_points():
    syms = _header_symbols()
    for need in ("ctct_b200_loss_forward", "ctct_b200_loss_backward", "ctct_b200_gather",
                 "ctct_b200_gathered_forward", "ctct_b200_workspace_bytes"):
        assert need in syms


def test_library_exports_every_declared_symbol(built):
    handle = ctypes.CDLL(built)
    for name in _header_symbols():
        assert hasattr(handle, name), name


def test_binding_covers_every_declared_symbol(built):
    from warp_ctct_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _header_symbols()
    lib = _lib.lib()
    assert lib.ctct_b200_abi_version() >= 1
    assert lib.ctct_b200_strerror(0) == b"ok"


def test_workspace_and_buffer_sizes(built):
    from warp_ctct_b200 import _lib
    lib = _lib.lib()
    assert lib.ctct_b200_grads3_elems(32, 256, 65) == 32 * 256 * 65 * 4
    small = lib.ctct_b200_workspace_bytes(32, 256, 65, 0)
    big = lib.ctct_b200_workspace_bytes(32, 256, 65, 1)
    assert 32 * 256 * 65 * 16 <= small < big
    assert big % 256 == 0
    assert lib.ctct_b200_workspace_bytes(4, 16, 9000, 1) == 0  # more contexts than the kernels support
    # the limit is where one staged pair of lattice rows stops fitting shared memory (CTCT_MAX_U1):
    # sizes beyond it are refused here, before a forward call could launch half its kernels
    header = open(os.path.join(ROOT, "include", "ctct_b200.h")).read()
    max_u1 = int(re.search(r"#define CTCT_MAX_U1 (\d+)", header).group(1))
    assert lib.ctct_b200_workspace_bytes(1, 4, max_u1, 1) > 0
    assert lib.ctct_b200_workspace_bytes(1, 4, max_u1 + 1, 1) == 0
    assert lib.ctct_b200_loss_forward(None, 0, None, None, None, 1, 4, max_u1 + 1, 5, 0, None, None, None, 0, None) != 0
    assert lib.ctct_b200_workspace_bytes(-1, 16, 5, 1) == 0


def test_argument_errors_do_not_need_a_gpu(built):
    from warp_ctct_b200 import _lib
    lib = _lib.lib()
    # null pointers / bad dtype are rejected before anything is launched
    assert lib.ctct_b200_loss_forward(None, 0, None, None, None, 2, 4, 3, 5, 0, None, None, None, 0, None) == -1
    assert lib.ctct_b200_loss_backward(None, None, None, None, None, 2, 4, 3, 5, 7, None, None) == -1
    assert lib.ctct_b200_gather(None, 9, None, None, None, 2, 4, 3, 5, 0, None, None) == -1
    with pytest.raises(RuntimeError):
        _lib.check(-2, "x")


def test_python_surface_matches_reference_signatures():
    import warp_ctct_b200 as W
    assert W.__all__ == ["ctct_loss", "ctct_simple_loss"]
    p = inspect.signature(W.ctct_loss).parameters
    assert list(p) == ["log_probs", "labels", "frames_lengths", "labels_lengths", "reduction", "average_frames"]
    assert p["reduction"].default == "mean" and p["average_frames"].default is False
    p = inspect.signature(W.ctct_simple_loss).parameters
    assert list(p) == ["f", "g", "labels", "frames_lengths", "labels_lengths", "reduction", "average_frames",
                       "normalized"]
    assert p["normalized"].default is True
    for cls in ("CTCTLoss", "LogMMExp", "SimpleCTCTLoss"):
        assert hasattr(W, cls)
    for fn in ("ctct_loss_fwd", "ctct_loss_simple_fwd", "log_matmul", "log_matmul_backward"):
        assert callable(getattr(W, fn))  # the four entry points of the reference's extension module


def test_cpu_tensors_are_rejected_like_the_reference():
    import torch
    import warp_ctct_b200 as W
    lp = torch.randn(2, 4, 3, 5).log_softmax(-1)
    ys = torch.ones(2, 2, dtype=torch.int32)
    lens = torch.tensor([4, 4], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="must be located in the CUDA"):
        W.ctct_loss(lp, ys, lens, torch.tensor([2, 2], dtype=torch.int32))
    with pytest.raises(AssertionError):
        W.ctct_loss(lp, ys[:, :1], lens, lens)
    with pytest.raises(AssertionError):
        W.ctct_loss(lp, ys, lens, lens, reduction="avg")


def test_import_level_drop_in():
    """`import warp_ctct` and `warp_ctct._C` resolve to this library with the reference's names."""
    import warp_ctct
    import warp_ctct._C as core
    import warp_ctct_b200 as W
    assert warp_ctct.ctct_loss is W.ctct_loss and warp_ctct.ctct_simple_loss is W.ctct_simple_loss
    assert warp_ctct.__all__ == ["ctct_loss", "ctct_simple_loss"] and warp_ctct.__version__ == W.__version__
    for cls in ("CTCTLoss", "LogMMExp", "SimpleCTCTLoss"):
        assert getattr(warp_ctct, cls) is getattr(W, cls)
    for fn in ("ctct_loss_fwd", "ctct_loss_simple_fwd", "log_matmul", "log_matmul_backward"):
        assert getattr(core, fn) is getattr(W, fn)
    # the reference's call shape: ctct_loss_simple_fwd(f, g, ys, den, lx, ly, requires_grad)
    assert list(inspect.signature(core.ctct_loss_simple_fwd).parameters) == ["f", "g", "ys", "den", "lx", "ly", "requires_grad"]
    assert list(inspect.signature(core.ctct_loss_fwd).parameters) == ["log_probs", "ys", "lx", "ly", "requires_grad"]
