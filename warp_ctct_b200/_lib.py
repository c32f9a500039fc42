"""ctypes binding of libctct_b200.so (the C ABI declared in include/ctct_b200.h).

There is no fallback of any kind: if the library is missing, cannot be loaded or reports an
error, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libctct_b200.so")

F32, F16, BF16 = 0, 1, 2
_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_lib = None

_vp, _i64, _int, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t

# name -> (restype, argtypes); must list every symbol of include/ctct_b200.h
SIGNATURES = {
    "ctct_b200_abi_version": (_int, []),
    "ctct_b200_strerror": (C.c_char_p, [_int]),
    "ctct_b200_grads3_elems": (_sz, [_i64, _i64, _i64]),
    "ctct_b200_workspace_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "ctct_b200_loss_forward": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp, _sz, _vp]),
    "ctct_b200_loss_forward_noalloc": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp]),
    "ctct_b200_loss_backward": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp]),
    "ctct_b200_loss_forward_reduced": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int, _int,
                                              C.c_float, _vp, _vp, _vp, _vp, _sz, _vp]),
    "ctct_b200_loss_forward_fused": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int, _int, C.c_float,
                                            _vp, _vp, _vp, _vp, _sz, _vp, _sz, _vp]),
    "ctct_b200_loss_backward_reduced": (_int, [_vp, _vp, _int, _int, C.c_float, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                               _int, _vp, _vp]),
    "ctct_b200_zero_fill": (_int, [_vp, _sz, _vp]),
    "ctct_b200_loss_backward_patch": (_int, [_vp, _vp, _int, _int, _int, C.c_float, _vp, _vp, _vp, _i64, _i64, _i64,
                                             _i64, _int, _vp, _vp]),
    "ctct_b200_logits_forward": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int, _int, C.c_float,
                                        _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "ctct_b200_logits_backward": (_int, [_vp, _vp, _int, _int, _int, C.c_float, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                         _i64, _int, _vp, _int, _vp]),
    "ctct_b200_packed_offsets": (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "ctct_b200_loss_forward_packed": (_int, [_vp, _int, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int, _int,
                                             C.c_float, _vp, _vp, _vp, _vp, _sz, _vp, _sz, _vp]),
    "ctct_b200_loss_backward_packed": (_int, [_vp, _vp, _int, _int, _int, C.c_float, _vp, _i64, _vp, _vp, _vp, _i64, _i64,
                                              _i64, _i64, _int, _vp, _vp]),
    "ctct_b200_logits_forward_packed": (_int, [_vp, _int, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int, _int,
                                               C.c_float, _vp, _vp, _vp, _vp, _sz, _vp]),
    "ctct_b200_logits_backward_packed": (_int, [_vp, _vp, _int, _int, _int, C.c_float, _vp, _vp, _i64, _vp, _vp, _vp, _i64,
                                                _i64, _i64, _i64, _int, _vp, _vp]),
    "ctct_b200_gather": (_int, [_vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp]),
    "ctct_b200_gather_probe": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int, _vp, _vp]),
    "ctct_b200_gathered_forward": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _sz, _vp]),
    "ctct_b200_export_tables": (_int, [_vp, _sz, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "ctct_b200_log_matmul": (_int, [_vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _vp]),
    "ctct_b200_log_matmul_tc_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64]),
    "ctct_b200_debug_set_wait_limit": (_int, [C.c_longlong]),
    "ctct_b200_log_matmul_tc_flags_offset": (_sz, [_i64, _i64, _i64, _i64]),
    "ctct_b200_log_matmul_tc": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _sz, _vp]),
    "ctct_b200_log_matmul_backward": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp]),
    "ctct_b200_log_matmul_backward_tc": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _sz, _vp]),
    "ctct_b200_simple_forward": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp, _sz, _vp]),
    "ctct_b200_simple_gathered_workspace_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "ctct_b200_simple_gathered_forward": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp,
                                                 _vp, _sz, _vp]),
    "ctct_b200_simple_backward": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp]),
    "ctct_b200_simple_backward_tc": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp,
                                            _sz, _vp]),
    "ctct_b200_profile_enable": (_int, [_int]),
    "ctct_b200_profile_read": (_int, [_vp, _vp, _int]),
    "ctct_b200_profile_disable": (_int, []),
}


def lib():
    """Load the shared library once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m warp_ctct_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().ctct_b200_strerror(rc).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {rc})")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {dtype}: expected float32, float16 or bfloat16") from None


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def raw_stream(device) -> int:
    """The current stream of `device` as an integer, without building a torch.cuda.Stream object."""
    return torch._C._cuda_getCurrentRawStream(device.index)


class on_device:
    """`with on_device(dev):` makes `dev` the current CUDA device; costs nothing when it already is
    (torch.cuda.device() takes ~10 microseconds per use, a tenth of a whole step of the loss)."""

    __slots__ = ("index", "prev")

    def __init__(self, device):
        self.index = device.index

    def __enter__(self):
        self.prev = torch.cuda.current_device()
        if self.prev != self.index:
            torch.cuda.set_device(self.index)
        return self

    def __exit__(self, *exc):
        if self.prev != self.index:
            torch.cuda.set_device(self.prev)
        return False


def workspace(N: int, T: int, U1: int, want_grad: bool, device) -> torch.Tensor:
    nbytes = lib().ctct_b200_workspace_bytes(N, T, U1, int(want_grad))
    if nbytes == 0 and N > 0:
        raise RuntimeError(f"unsupported problem size N={N}, T={T}, U+1={U1}")
    # torch's caching allocator hands out blocks aligned to 512 bytes
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
