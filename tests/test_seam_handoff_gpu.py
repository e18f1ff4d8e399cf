"""The forward kernel's second way of getting the carry across a seam: handed over between CTAs of a thread-block
cluster through distributed shared memory (BTP_SEAM_HANDOFF), as the reference does between the CTAs of its cluster
(csrc/btp/btp-forward.cu:276-335), instead of recomputed from the block to the left (the default).

Checked here, through the C ABI: the hand-off is really taken (cluster size of the launch), its result agrees with
the oracle and, to rounding, with the recomputing kernel for every cluster size (1, 2, 4, 8 CTAs) and coefficient
form; calls it does not cover fall back to recomputing; and a hand-off that never arrives is given up after the
wait limit and reported, with nothing hanging."""

from __future__ import annotations

import ctypes

import pytest
import torch

import btp_oracle as O

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _inputs(B, H, L, kind, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, H, 16, L, generator=g).to(dtype).cuda()
    if kind == "16bit":
        a, tag = torch.sigmoid(torch.randn(B, H, L, generator=g) + 2).to(dtype).cuda(), None
    elif kind == "f32":
        a, tag = torch.sigmoid(torch.randn(B, H, L, generator=g) + 2).cuda(), 1
    else:
        a, tag = (-1e-3 * torch.rand(B, H, L, generator=g)).cuda(), 2
    return a, x, tag


def _forward(lib, a, x, tag, k=2, y_dtype=None, ckpt=None):
    from spear_b200 import _lib

    B, H, _, L = x.shape
    f16 = x.dtype == torch.float16
    act = _lib.DTYPE_F16 if f16 else _lib.DTYPE_BF16
    ctag = act if tag is None else (tag | (_lib.ACT_F16 if f16 else 0))
    y = torch.full(x.shape, float("nan"), device="cuda", dtype=y_dtype or x.dtype)
    ytag = _lib.DTYPE_F32 if y.dtype == torch.float32 else act
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.btp_sm100_forward(_ptr(a), _ptr(x), _ptr(y), None if ckpt is None else _ptr(ckpt), B, H, L, k, ctag, ytag, stream)
    assert rc == 0, lib.btp_sm100_last_error().decode()
    torch.cuda.synchronize()
    return y


@pytest.fixture()
def handoff():
    from spear_b200 import _lib

    lib = _lib.load()
    previous = _lib.set_seam_mode(_lib.SEAM_HANDOFF)
    try:
        yield lib
    finally:
        _lib.set_seam_mode(previous)
        _lib.device_status()


# B, H, L, coefficient form, activations, expected cluster size.  A shape qualifies when it gives every warp of
# the full grid at least four stretches, hence the large batches at short L.
CASES = [
    (4736, 1, 512, "16bit", torch.bfloat16, 1),    # 2 stretches per sequence, both inside one CTA
    (37, 64, 1024, "f32", torch.bfloat16, 1),      # 4 stretches = the 4 warps of one CTA
    (1184, 1, 2048, "16bit", torch.bfloat16, 2),
    (16, 37, 4096, "f32log", torch.bfloat16, 4),
    (16, 64, 8192, "f32log", torch.bfloat16, 4),   # the long-sequence benchmark configuration
    (16, 64, 8192, "16bit", torch.float16, 4),
    (8, 37, 16384, "16bit", torch.bfloat16, 8),
]


@pytest.mark.parametrize("B,H,L,kind,dtype,cluster", CASES)
def test_handoff_matches_the_oracle_and_the_recomputing_kernel(handoff, B, H, L, kind, dtype, cluster):
    from spear_b200 import _lib

    lib = handoff
    a, x, tag = _inputs(B, H, L, kind, dtype, seed=L + B)
    y_h = _forward(lib, a, x, tag)
    grid, got_cluster = _lib.last_launch()
    assert got_cluster == cluster and grid % cluster == 0
    _lib.device_status()
    _lib.set_seam_mode(_lib.SEAM_RECOMPUTE)
    y_r = _forward(lib, a, x, tag)
    assert _lib.last_launch()[1] == 1
    _lib.set_seam_mode(_lib.SEAM_HANDOFF)
    assert torch.isfinite(y_h.float()).all()
    # the two kernels differ only in how the 16 numbers at a seam are summed (tensor-core product of the run's
    # last block against fp32 FMAs over the re-read block): a handful of outputs land on the other side of a rounding
    diff = (y_h.float() - y_r.float()).norm() / y_r.float().norm()
    assert diff <= 2e-5, diff
    assert (y_h != y_r).float().mean() <= 1e-4
    # against the oracle, on the first and the last sequences of the batch (all their seams)
    sel = [0, B - 1]
    af = a[sel].float().cpu()
    want = O.btp_forward(torch.exp(af) if kind == "f32log" else af, x[sel].float().cpu())
    rel_h = O.rel_l2(y_h[sel].float().cpu(), want)
    rel_r = O.rel_l2(y_r[sel].float().cpu(), want)
    assert rel_h <= 1e-2 and rel_h <= rel_r * 1.01 + 1e-6, (rel_h, rel_r)
    # bitwise repeatable although the hand-off's timing is not
    assert torch.equal(_forward(lib, a, x, tag), y_h)


def test_calls_the_handoff_does_not_cover_recompute(handoff):
    from spear_b200 import _lib

    lib = handoff
    a, x, tag = _inputs(16, 37, 4096, "16bit", torch.bfloat16, seed=3)
    want = O.btp_forward(a[:1].float().cpu(), x[:1].float().cpu())
    y = _forward(lib, a, x, tag)
    assert _lib.last_launch()[1] == 4
    # float32 output, a checkpoint, k = 1, a ragged length, too few sequences: the recomputing kernel runs
    y32 = _forward(lib, a, x, tag, y_dtype=torch.float32)
    assert _lib.last_launch()[1] == 1
    assert O.rel_l2(y32[:1].cpu(), want) <= 1e-2
    ck = torch.zeros(16, 37, 4096 // 16, 16, device="cuda")
    yc = _forward(lib, a, x, tag, ckpt=ck)
    assert _lib.last_launch()[1] == 1 and torch.equal(yc, _forward_recompute(lib, a, x, tag))
    _forward(lib, a, x, tag, k=1)
    assert _lib.last_launch()[1] == 1
    a2, x2, _ = _inputs(16, 37, 4096 + 64, "16bit", torch.bfloat16, seed=4)
    _forward(lib, a2, x2, None)
    assert _lib.last_launch()[1] == 1
    a3, x3, _ = _inputs(2, 3, 4096, "16bit", torch.bfloat16, seed=5)
    _forward(lib, a3, x3, None)
    assert _lib.last_launch()[1] == 1
    assert O.rel_l2(y[:1].float().cpu(), want) <= 1e-2


def _forward_recompute(lib, a, x, tag):
    from spear_b200 import _lib

    _lib.set_seam_mode(_lib.SEAM_RECOMPUTE)
    try:
        return _forward(lib, a, x, tag)
    finally:
        _lib.set_seam_mode(_lib.SEAM_HANDOFF)


def test_a_handoff_that_never_arrives_is_given_up_and_reported(handoff):
    """Warp 0 of block 0 loses its first load (test hook) and gives up, so it never hands its carry on.  It sets the
    abort word of its cluster, the warps waiting for a hand-off down the chain give up with it, and the kernel ends
    after about ONE wait limit (not one per warp of the chain).  Nothing hangs, the context stays usable, the error
    is reported, and the next launch is right."""
    from spear_b200 import _lib

    lib = handoff
    a, x, tag = _inputs(16, 37, 4096, "16bit", torch.bfloat16, seed=9)
    detail = (ctypes.c_uint * 4)()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    limit_ms = 20
    previous = lib.btp_sm100_set_wait_limit(limit_ms * 1_000_000)
    try:
        lib.btp_sm100_test_expect_missing_bytes(64)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        _forward(lib, a, x, tag)
        t1.record()
        torch.cuda.synchronize()
        assert _lib.last_launch()[1] == 4
        # 16 warps share a sequence: one limit each down the chain would be 16 x 20 ms
        assert limit_ms <= t0.elapsed_time(t1) < 4 * limit_ms, t0.elapsed_time(t1)
        rc = lib.btp_sm100_device_status(stream, detail)
        assert rc == -8 and list(detail)[0] == 1 and list(detail)[1] == 0  # a timeout, in block 0
        assert lib.btp_sm100_device_status(stream, detail) == 0
        y = _forward(lib, a, x, tag)
        assert lib.btp_sm100_device_status(stream, detail) == 0
    finally:
        lib.btp_sm100_set_wait_limit(previous)
    want = O.btp_forward(a[:2].float().cpu(), x[:2].float().cpu())
    assert O.rel_l2(y[:2].float().cpu(), want) <= 1e-2
    assert torch.equal(y, _forward(lib, a, x, tag))
