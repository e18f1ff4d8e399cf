"""ctypes binding of libbtp_sm100.so (declared in include/btp_sm100.h).

There is no fallback of any kind: if the shared library is missing the import
of the ops fails with instructions to build it; if a call returns a non-zero
status a RuntimeError carries the library's own message.
"""

from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libbtp_sm100.so")

# dtype tags of include/btp_sm100.h
DTYPE_BF16 = 0
DTYPE_F32 = 1
DTYPE_F32_LOG = 2
DTYPE_F16 = 3
ACT_F16 = 0x10  # flag on a float coefficient tag: the activations are float16

SEAM_RECOMPUTE = 0  # forward: the carry across a seam is recomputed from the block to the left (default)
SEAM_HANDOFF = 1    # forward: the carry is handed over through distributed shared memory inside a cluster

ABI_VERSION = 4

# every symbol include/btp_sm100.h declares: name -> (restype, argtypes)
_vp, _i, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
SYMBOLS = {
    "btp_sm100_forward": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "btp_sm100_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "btp_sm100_forward_noalloc": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "btp_sm100_gated_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _ll, _i, _vp]),
    "btp_sm100_gated_backward": (_i, [_vp] * 9 + [_i, _i, _i, _i] + [_ll] * 9 + [_i, _vp]),
    "btp_sm100_decode_step": (_i, [_vp] * 11 + [_ll, _i, _i, _i, _i, _i, _vp]),
    "btp_sm100_prefill_state": (_i, [_vp] * 5 + [_ll, _i, _i, _i, _i, _vp]),
    "btp_sm100_noalloc_read_record": (_i, [_vp, _ll, _vp]),
    "btp_sm100_set_wait_limit": (ctypes.c_ulonglong, [ctypes.c_ulonglong]),
    "btp_sm100_set_seam_mode": (_i, [_i]),
    "btp_sm100_last_launch": (None, [ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "btp_sm100_test_expect_missing_bytes": (None, [ctypes.c_uint]),
    "btp_sm100_status_string": (ctypes.c_char_p, [_i]),
    "btp_sm100_last_error": (ctypes.c_char_p, []),
    "btp_sm100_device_status": (_i, [_vp, ctypes.POINTER(ctypes.c_uint)]),
    "btp_sm100_launch_count": (ctypes.c_ulonglong, []),
    "btp_sm100_abi_version": (_i, []),
}

_lock = threading.Lock()
_lib = None


class BtpLibraryError(RuntimeError):
    """The native library is missing, stale or reported an error."""


def load() -> ctypes.CDLL:
    """Loads the library once and declares the prototypes.  Never builds, never falls back."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise BtpLibraryError(
                f"{LIB_PATH} is missing. Build it with `python -m spear_b200.build` "
                "(needs nvcc; the BTP ops have no CPU or PyTorch fallback)."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(lib, name)  # AttributeError here = stale library
            fn.restype = restype
            fn.argtypes = argtypes
        if lib.btp_sm100_abi_version() != ABI_VERSION:
            raise BtpLibraryError(
                f"{LIB_PATH} has ABI version {lib.btp_sm100_abi_version()}, expected {ABI_VERSION}; rebuild it."
            )
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    """Raises RuntimeError for a non-zero status, with the library's own text."""
    if status == 0:
        return
    lib = load()
    name = lib.btp_sm100_status_string(status).decode()
    detail = lib.btp_sm100_last_error().decode()
    raise RuntimeError(f"{what} failed: {name}: {detail}")


def device_status(stream: int = 0) -> None:
    """Synchronises `stream` and raises if a kernel's bounded wait gave up."""
    lib = load()
    detail = (ctypes.c_uint * 4)()
    check(lib.btp_sm100_device_status(ctypes.c_void_p(stream), detail), "btp_sm100_device_status")


def set_seam_mode(mode: int) -> int:
    """Selects how the forward kernel gets the carry across a seam (SEAM_RECOMPUTE, SEAM_HANDOFF); process-wide.
    Returns the previous mode."""
    if mode not in (SEAM_RECOMPUTE, SEAM_HANDOFF):
        raise ValueError(f"seam mode must be SEAM_RECOMPUTE (0) or SEAM_HANDOFF (1), got {mode!r}")
    return int(load().btp_sm100_set_seam_mode(mode))


def last_launch() -> tuple[int, int]:
    """(CTAs, cluster size) of the last forward/backward kernel this thread launched."""
    g, c = _i(0), _i(0)
    load().btp_sm100_last_launch(ctypes.byref(g), ctypes.byref(c))
    return g.value, c.value


def launch_count() -> int:
    return int(load().btp_sm100_launch_count())
