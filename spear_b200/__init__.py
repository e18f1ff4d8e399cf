"""spear_b200: the block two-pass (BTP) hot path of SPEAR, hand-written for NVIDIA B200 (sm_100a).

    from spear_b200.ops.btp import btp          # same signature as spear.ops.btp.btp
    from spear_b200.nn.phalanx import Phalanx   # same constructor / state_dict as spear.nn.phalanx.Phalanx

The native library is loaded on first use; there is no CPU or PyTorch fallback.
"""

__version__ = "0.1.0"

__all__ = ["btp", "Phalanx", "SigmoidA", "install_as_spear_backend"]


def install_as_spear_backend():
    """Makes an UNMODIFIED installation of the reference package `spear` run on these kernels.

    Registers `spear_b200._btp` as the compiled extension module `spear._btp` that the reference imports
    (spear/ops/btp/interface.py:16) and calls (interface.py:63,87).  Call it before or after `import spear`.
    Returns the imported `spear` package.
    """
    import importlib
    import sys

    from . import _btp as native

    sys.modules["spear._btp"] = native
    spear = importlib.import_module("spear")
    spear._btp = native  # `spear._btp.forward(...)` is looked up as an attribute at call time
    return spear


def __getattr__(name):  # lazy: importing the package must not require torch ops to be registered
    if name == "btp":
        from .ops.btp import btp

        return btp
    if name in ("Phalanx", "SigmoidA"):
        from .nn import phalanx

        return getattr(phalanx, name)
    raise AttributeError(name)
