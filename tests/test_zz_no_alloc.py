"""`btp_sm100_forward_noalloc`: the forward for callers that can hand over nothing but their input and
output buffers (a serving process whose memory all belongs to a start-up arena, a plugin that is not
allowed to call the CUDA allocator).  The carry record that `btp_sm100_forward` writes to a buffer of
the caller's goes to a fixed 4 MiB array inside the library instead.

Checked here, straight through the C ABI: its y equals the y of the ordinary entry point on two calls in
a row (different sizes, so the second call runs over whatever the first one left in the shared array), the
record it leaves in the array equals the checkpoint of the ordinary entry point on both calls, and a
problem larger than the array is refused with BTP_ERR_TOO_LARGE.  This file sorts last on purpose:
a run that stops at the first failure has then already run every other test."""

from __future__ import annotations

import ctypes

import pytest
import torch

import btp_oracle as O

pytestmark = pytest.mark.gpu

MAX_HEAD_TOKENS = 1 << 20  # BTP_SM100_NOALLOC_MAX_HEAD_TOKENS in include/btp_sm100.h


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _inputs(B, H, L, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(B, H, 16, L, generator=g) * 0.5).bfloat16().cuda()
    a = torch.sigmoid(torch.randn(B, H, L, generator=g)).bfloat16().cuda()
    return a, x


def test_noalloc_forward_matches_forward_twice_in_a_row():
    from spear_b200 import _lib

    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for B, H, L, seed in ((8, 16, 512, 21), (3, 5, 208, 22)):  # second call: smaller and ragged
        a, x = _inputs(B, H, L, seed)
        y_ref = torch.full_like(x, float("nan"))
        ckpt = torch.empty(B, H, L // 16, 16, device="cuda", dtype=torch.float32)
        _lib.check(lib.btp_sm100_forward(_ptr(a), _ptr(x), _ptr(y_ref), _ptr(ckpt), B, H, L, 2, 0, 0, stream), "forward")
        y_new = torch.full_like(x, float("nan"))
        _lib.check(lib.btp_sm100_forward_noalloc(_ptr(a), _ptr(x), _ptr(y_new), B, H, L, 2, 0, 0, stream), "forward_noalloc")
        torch.cuda.synchronize()
        _lib.device_status()
        assert torch.isfinite(y_new.float()).all()
        # same kernel, same inputs: the tolerance of the parity tests is met with room to spare
        assert O.rel_l2(y_new.float().cpu(), y_ref.float().cpu()) <= 1e-2
        assert O.rel_l2(y_new.float().cpu(), O.btp_forward(a.float().cpu(), x.float().cpu())) <= 1e-2
        # The record itself: y does not depend on it, so read the built-in array back and compare it with the
        # checkpoint the ordinary entry point wrote for the same inputs (every slot but the last of a sequence,
        # which neither entry point writes).  A kernel that had been handed a wrong address would fail here.
        nb = L // 16
        record = torch.full((B, H, nb, 16), float("nan"), device="cuda", dtype=torch.float32)
        _lib.check(lib.btp_sm100_noalloc_read_record(_ptr(record), record.numel(), stream), "noalloc_read_record")
        torch.cuda.synchronize()
        assert torch.equal(record[:, :, : nb - 1], ckpt[:, :, : nb - 1])
        assert record[:, :, : nb - 1].abs().sum().item() > 0


def test_noalloc_forward_without_carry_ignores_the_limit():
    """k = 1 writes no record, so a problem larger than the built-in array is accepted."""
    from spear_b200 import _lib

    lib = _lib.load()
    B, H, L = 9, 1024, 128  # 1 179 648 head-tokens > 2^20
    assert B * H * L > MAX_HEAD_TOKENS
    a, x = _inputs(B, H, L, 24)
    y_ref, y_new = torch.empty_like(x), torch.empty_like(x)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.btp_sm100_forward(_ptr(a), _ptr(x), _ptr(y_ref), None, B, H, L, 1, 0, 0, stream), "forward")
    _lib.check(lib.btp_sm100_forward_noalloc(_ptr(a), _ptr(x), _ptr(y_new), B, H, L, 1, 0, 0, stream), "forward_noalloc")
    torch.cuda.synchronize()
    assert torch.equal(y_new, y_ref)


def test_noalloc_forward_refuses_what_does_not_fit():
    from spear_b200 import _lib

    lib = _lib.load()
    B, H, L = 1, 1, 16
    a, x = _inputs(B, H, L, 23)
    y = torch.empty_like(x)
    # sizes are checked before any pointer is used: B*H*L just over the limit
    big_b = MAX_HEAD_TOKENS // 128 + 1
    rc = lib.btp_sm100_forward_noalloc(_ptr(a), _ptr(x), _ptr(y), big_b, 1, 128, 2, 0, 0, ctypes.c_void_p(0))
    assert rc == -9 and lib.btp_sm100_status_string(rc).decode() == "BTP_ERR_TOO_LARGE"
    assert "exceeds the built-in scratch" in lib.btp_sm100_last_error().decode()
    # exactly at the limit is accepted as far as the size check goes (tiny real call afterwards still works)
    _lib.check(lib.btp_sm100_forward_noalloc(_ptr(a), _ptr(x), _ptr(y), B, H, L, 2, 0, 0, ctypes.c_void_p(0)), "forward_noalloc")
    torch.cuda.synchronize()
    assert O.rel_l2(y.float().cpu(), O.btp_forward(a.float().cpu(), x.float().cpu())) <= 1e-2
