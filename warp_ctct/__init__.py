"""Import-level drop-in: ``from warp_ctct import ctct_loss, ctct_simple_loss`` keeps working.

Code written against maxwellzh/warp-ctct imports the package ``warp_ctct`` (and, for the extension
functions, ``warp_ctct._C``; setup.py:26 of that project builds it).  This package has no code of
its own: every name is the B200 implementation in ``warp_ctct_b200``.
"""
from warp_ctct_b200 import (CTCTLoss, LogMMExp, SimpleCTCTLoss, __version__, ctct_loss,  # noqa: F401
                            ctct_loss_from_logits, ctct_simple_loss)

from . import _C  # noqa: F401

__all__ = ["ctct_loss", "ctct_simple_loss"]
