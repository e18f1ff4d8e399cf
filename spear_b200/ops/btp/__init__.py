"""Block two-pass (BTP) operator on the sm_100a kernels (mirror of spear.ops.btp)."""

from .interface import btp

__all__ = ["btp"]
