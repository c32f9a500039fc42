"""The four functions the reference's extension module exports (csrc/binding.cpp:326-345), bound to
the C ABI of libctct_b200.so through ``warp_ctct_b200``: same names, arguments, results and errors."""
from warp_ctct_b200 import ctct_loss_fwd, ctct_loss_simple_fwd, log_matmul, log_matmul_backward  # noqa: F401

__all__ = ["ctct_loss_fwd", "ctct_loss_simple_fwd", "log_matmul", "log_matmul_backward"]
