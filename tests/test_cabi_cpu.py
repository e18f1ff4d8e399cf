"""The C-ABI library on a machine without a GPU: it loads, exports every symbol that
include/btp_sm100.h declares, names its status codes, and rejects bad arguments before
touching CUDA.  No compute call is made."""

from __future__ import annotations

import ctypes
import os
import re

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "btp_sm100.h")


@pytest.fixture(scope="module")
def lib():
    from spear_b200 import _lib, build

    build.build()  # no-op when the library is up to date
    return _lib.load()


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(btp_sm100_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from spear_b200 import _lib

    names = declared_functions()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/btp_sm100.h but not exported"
    assert sorted(_lib.SYMBOLS) == names, "the ctypes prototypes and the header disagree"


def test_abi_version_and_status_strings(lib):
    assert lib.btp_sm100_abi_version() == 4
    seen = set()
    for code in range(0, -10, -1):
        name = lib.btp_sm100_status_string(code).decode()
        assert name.startswith("BTP_")
        seen.add(name)
    assert len(seen) == 10 and "BTP_OK" in seen
    assert lib.btp_sm100_status_string(-99).decode() == "BTP_ERR_UNKNOWN"
    text = open(HEADER).read()
    for name in seen:
        assert name in text


def test_seam_mode_and_launch_shape_are_host_state(lib):
    """btp_sm100_set_seam_mode returns the previous mode, ignores values it does not know, and the launch-shape
    diagnostic reads zeros on a thread that has launched nothing (no GPU is touched by either)."""
    from spear_b200 import _lib

    header = open(HEADER).read()
    assert "#define BTP_SEAM_RECOMPUTE 0" in header and "#define BTP_SEAM_HANDOFF 1" in header
    assert (_lib.SEAM_RECOMPUTE, _lib.SEAM_HANDOFF) == (0, 1)
    assert lib.btp_sm100_set_seam_mode(_lib.SEAM_HANDOFF) == _lib.SEAM_RECOMPUTE  # the default
    assert lib.btp_sm100_set_seam_mode(7) == _lib.SEAM_HANDOFF  # unknown value: nothing changes
    assert lib.btp_sm100_set_seam_mode(-1) == _lib.SEAM_HANDOFF
    assert _lib.set_seam_mode(_lib.SEAM_RECOMPUTE) == _lib.SEAM_HANDOFF
    assert lib.btp_sm100_set_seam_mode(_lib.SEAM_RECOMPUTE) == _lib.SEAM_RECOMPUTE
    with pytest.raises(ValueError):
        _lib.set_seam_mode(2)
    assert _lib.last_launch() == (0, 0)
    lib.btp_sm100_last_launch(None, None)  # either pointer may be NULL


def _fwd(lib, coeff=16, x=16, y=16, ck=0, B=1, H=1, L=16, k=2, cd=0, od=0):
    p = ctypes.c_void_p
    return lib.btp_sm100_forward(p(coeff), p(x), p(y), p(ck), B, H, L, k, cd, od, p(0))


def _bwd(lib, coeff=16, x=16, dy=16, dx=16, dA=16, B=1, H=1, L=16, k=2, cd=0, dd=0):
    p = ctypes.c_void_p
    return lib.btp_sm100_backward(p(coeff), p(x), p(dy), p(0), p(dx), p(dA), B, H, L, k, cd, dd, p(0))


def test_argument_errors_come_back_as_codes(lib):
    """Every check below fires before any CUDA call, so fake (never dereferenced) pointers are fine."""
    err = lambda: lib.btp_sm100_last_error().decode()
    assert _fwd(lib, L=24) == -2 and "multiple of 16" in err()       # BTP_ERR_BAD_SHAPE
    assert _fwd(lib, B=0) == -2
    assert _fwd(lib, H=-3) == -2
    assert _fwd(lib, k=3) == -3 and "k must be 1 or 2" in err()      # BTP_ERR_BAD_ORDER
    assert _fwd(lib, cd=7) == -4                                      # BTP_ERR_BAD_DTYPE
    assert _fwd(lib, od=2) == -4
    assert _fwd(lib, x=0) == -1                                       # BTP_ERR_NULL_POINTER
    assert _fwd(lib, y=8) == -5 and "aligned" in err()                # BTP_ERR_MISALIGNED
    assert _fwd(lib, ck=4) == -5
    assert _fwd(lib, B=1 << 20, H=1 << 10, L=16) == -2                # B*H*16 rows beyond int32
    assert _bwd(lib, L=8) == -2
    assert _bwd(lib, k=0) == -3
    assert _bwd(lib, dd=2) == -4
    assert _bwd(lib, dA=0) == -1
    assert _bwd(lib, dx=24) == -5


def test_dtype_tags_of_the_plain_entry_points(lib):
    """bfloat16 or float16 activations, chosen through the coefficient tag; y / dy float32 or the activations' type."""
    p = ctypes.c_void_p

    def fwd(ctag, otag):
        return lib.btp_sm100_forward(p(16), p(16), p(16), p(0), 1, 1, 16, 2, ctag, otag, p(0))

    def bwd(ctag, dtag):
        return lib.btp_sm100_backward(p(16), p(16), p(16), p(0), p(16), p(16), 1, 1, 16, 2, ctag, dtag, p(0))

    BF16, F32, LOG, F16, ACT = 0, 1, 2, 3, 0x10
    for call in (fwd, bwd):
        assert call(BF16 | ACT, F32) == -4 and "bfloat16 coefficient cannot go with float16" in lib.btp_sm100_last_error().decode()
        assert call(4, F32) == -4 and call(0x20, F32) == -4          # unknown tag, unknown flag
        assert call(BF16, F16) == -4 and call(F16, BF16) == -4        # 16-bit y / dy of the other type
        assert call(F32 | ACT, BF16) == -4 and call(LOG, F16) == -4
        # valid combinations get past the dtype checks (and fail later only for want of a GPU, or succeed)
        for ctag, otag in ((BF16, BF16), (BF16, F32), (F32, BF16), (LOG, F32), (F16, F16), (F16, F32), (F32 | ACT, F16), (LOG | ACT, F32)):
            assert call(ctag, otag) != -4, (ctag, otag)


def test_gated_entry_points_check_their_arguments(lib):
    p, ll = ctypes.c_void_p, ctypes.c_longlong

    def fwd(B=1, L=16, H=4, k=2, ld=(4, 64, 64, 64, 64), ptrs=(16, 16, 16, 16, 16), kv=None):
        return lib.btp_sm100_gated_forward(*[p(x) for x in ptrs], B, L, H, H if kv is None else kv, *[ll(x) for x in ld], k, p(0))

    def bwd(B=1, L=16, H=4, k=2, ld=(4, 64, 64, 64, 64, 4, 64, 64, 64), ptrs=(16,) * 9, kv=None):
        return lib.btp_sm100_gated_backward(*[p(x) for x in ptrs], B, L, H, H if kv is None else kv, *[ll(x) for x in ld], k, p(0))

    assert fwd(kv=3) == -2 and "kv_heads must divide" in lib.btp_sm100_last_error().decode()
    assert fwd(kv=0) == -2 and bwd(kv=3) == -2
    assert fwd(kv=2, ld=(4, 24, 32, 64, 64)) == -2   # shared heads: B_logits row narrower than kv_heads*16
    assert bwd(kv=2, ld=(4, 32, 32, 64, 64, 4, 24, 64, 64)) == -2   # groups of 2 are summed in the kernel: dB_logits has H*16/2 columns
    assert bwd(kv=2, ld=(4, 32, 32, 64, 64, 4, 32, 32, 64)) != -2   # ... and a pitch of exactly that passes the shape checks

    assert fwd(H=6) == -2 and "multiple of 4" in lib.btp_sm100_last_error().decode()
    assert fwd(L=24) == -2
    assert fwd(k=0) == -3
    assert fwd(ptrs=(16, 0, 16, 16, 16)) == -1
    assert fwd(ld=(4, 60, 64, 64, 64)) == -2      # pitch smaller than the row
    assert fwd(ld=(4, 68, 64, 64, 64)) == -5      # pitch not a multiple of 8 elements
    assert fwd(ptrs=(16, 8, 16, 16, 16)) == -5
    assert bwd(H=2) == -2
    assert bwd(L=8) == -2
    assert bwd(k=3) == -3
    assert bwd(ptrs=(16,) * 8 + (0,)) == -1
    assert bwd(ld=(4, 64, 64, 64, 64, 6, 64, 64, 64)) == -5
    assert bwd(ptrs=(16, 16, 16, 16, 16, 4, 16, 16, 16)) == -5


def test_streaming_entry_points_check_their_arguments(lib):
    p, ll = ctypes.c_void_p, ctypes.c_longlong

    def step(ptrs=(16,) * 11, n=4, done=0, dtype=1, gdtype=1):
        return lib.btp_sm100_decode_step(*[p(x) for x in ptrs], ll(n), done, 0, 0, dtype, gdtype, p(0))

    def state(ptrs=(16,) * 5, n=4, L=20, dtype=0, gdtype=1):
        return lib.btp_sm100_prefill_state(*[p(x) for x in ptrs], ll(n), L, 0, dtype, gdtype, p(0))

    err = lambda: lib.btp_sm100_last_error().decode()
    assert step(n=0) == -2
    assert step(dtype=2) == -4 and step(gdtype=5) == -4
    assert step(ptrs=(16, 0) + (16,) * 9) == -1
    assert step(ptrs=(16,) * 10 + (0,), done=1) == -1 and "completes a block" in err()
    assert step(ptrs=(16, 8) + (16,) * 9) == -5
    assert step(ptrs=(2,) + (16,) * 10) == -5          # float gate on a 2-byte boundary
    assert state(L=0) == -2 and state(n=-1) == -2
    assert state(dtype=2) == -4
    assert state(ptrs=(16, 16, 0, 16, 16)) == -1
    assert state(ptrs=(2, 16, 16, 16, 16)) == -5


def test_no_gpu_is_an_error_not_a_fallback(lib):
    """With valid arguments and no usable device the call fails with a CUDA error code; nothing is computed."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    rc = _fwd(lib)
    assert rc in (-6, -7)
    assert lib.btp_sm100_last_error().decode() != ""
    assert lib.btp_sm100_launch_count() == 0


def test_python_wrapper_has_no_cpu_path():
    import torch

    from spear_b200.nn.phalanx import Phalanx
    from spear_b200.ops.btp import btp

    with pytest.raises(RuntimeError, match="no CPU path"):
        btp(torch.rand(1, 2, 32), torch.rand(1, 2, 16, 32))
    for method in ("pytorch", "pytorch_linspace"):
        with pytest.raises(NotImplementedError):
            Phalanx(dim=32, method=method)
    with pytest.raises(ValueError):
        Phalanx(dim=32, method="triton")
    with pytest.raises(ValueError):
        Phalanx(dim=40)            # not divisible by 16 (swr.py:241-242)
    with pytest.raises(ValueError):
        Phalanx(dim=64, heads=2)   # head_dim must be 16 (swr.py:247-249)
    with pytest.raises(ValueError):
        Phalanx(dim=64, kv_heads=3)


def test_gated_wrappers_refuse_mismatched_shapes_before_any_launch():
    """The gated kernels size their descriptors from a_logits alone; a tensor with fewer tokens or batch entries
    must be refused on the host (ValueError), never reach a launch."""
    import torch

    from spear_b200 import _lib
    from spear_b200.ops.btp import gated

    B, L, H = 2, 32, 4
    mk = lambda b, l, c: torch.zeros(b, l, c, dtype=torch.bfloat16)
    al, bl, c, v, out = mk(B, L, H), mk(B, L, 64), mk(B, L, 64), mk(B, L, 64), mk(B, L, 64)
    before = _lib.launch_count() if os.path.exists(_lib.LIB_PATH) else 0
    for bad in (dict(v=mk(B, L - 16, 64)), dict(c=mk(B - 1, L, 64)), dict(out=mk(B, L // 2, 64)), dict(bl=mk(B, 2 * L, 64))):
        args = {**dict(al=al, bl=bl, c=c, v=v, out=out), **bad}
        with pytest.raises(ValueError, match="batch and length"):
            gated._launch_forward(args["al"], args["bl"], args["c"], args["v"], args["out"], 2)
    grads = [mk(B, L, H)] + [mk(B, L, 64) for _ in range(3)]
    for i in range(4):
        g = list(grads)
        g[i] = mk(B, L + 16, g[i].shape[2])
        with pytest.raises(ValueError, match="batch and length"):
            gated._launch_backward(al, bl, c, v, out, *g, 2)
    with pytest.raises(ValueError, match="batch and length"):
        gated._launch_backward(al, bl, c, v, mk(B, L - 16, 64), *grads, 2)
    if os.path.exists(_lib.LIB_PATH):
        assert _lib.launch_count() == before
