"""Block two-pass (BTP) operator on the sm_100a kernels (mirror of spear.ops.btp)."""

from .host import btp_fwd_bwd_host
from .interface import btp

__all__ = [
    "btp",
    "btp_fwd_bwd_host",
]
