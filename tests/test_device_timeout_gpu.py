"""The give-up path of the kernels' bounded waits, exercised without faulting or hanging anything.

Every wait inside the forward and backward kernels is on the warp's own loads and is bounded
(btp_sm100_set_wait_limit, default 2 s).  Here the bound is shortened to 1 ms and the test hook
btp_sm100_test_expect_missing_bytes makes ONE warp of the next launch expect bytes that no copy delivers, so
that exactly one wait runs out.  Expected: the kernel returns normally, the context stays usable,
btp_sm100_device_status reports BTP_ERR_DEVICE_TIMEOUT once with the block and warp, then reads clean again,
every other warp's output is correct, and the next launch is correct everywhere."""

from __future__ import annotations

import ctypes

import pytest
import torch

import btp_oracle as O

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("which", ["forward", "backward"])
def test_a_wait_that_runs_out_is_reported_once_and_the_context_stays_usable(which):
    from spear_b200 import _lib

    lib = _lib.load()
    _lib.device_status()  # start clean
    g = torch.Generator().manual_seed(5)
    B, H, L = 4, 8, 256
    a = torch.sigmoid(torch.randn(B, H, L, generator=g)).bfloat16().cuda()
    x = torch.randn(B, H, 16, L, generator=g).bfloat16().cuda()
    dy = torch.randn(B, H, 16, L, generator=g).bfloat16().cuda()
    y_w = O.btp_forward(a.float().cpu(), x.float().cpu())
    dA_w, dx_w = O.btp_backward(a.float().cpu(), x.float().cpu(), dy.float().cpu())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def launch():
        if which == "forward":
            out = torch.full_like(x, float("nan"))
            rc = lib.btp_sm100_forward(_ptr(a), _ptr(x), _ptr(out), None, B, H, L, 2, 0, 0, stream)
            aux = None
        else:
            out = torch.full_like(x, float("nan"))
            aux = torch.full((B, H, L), float("nan"), device="cuda")
            rc = lib.btp_sm100_backward(_ptr(a), _ptr(x), _ptr(dy), None, _ptr(out), _ptr(aux), B, H, L, 2, 0, 0, stream)
        assert rc == 0, lib.btp_sm100_last_error().decode()
        torch.cuda.synchronize()
        return out, aux

    want = y_w if which == "forward" else dx_w
    previous = lib.btp_sm100_set_wait_limit(1_000_000)  # 1 ms
    try:
        lib.btp_sm100_test_expect_missing_bytes(64)
        out, _ = launch()  # returns: nothing hangs
        detail = (ctypes.c_uint * 4)()
        rc = lib.btp_sm100_device_status(stream, detail)
        assert rc == -8 and lib.btp_sm100_status_string(rc).decode() == "BTP_ERR_DEVICE_TIMEOUT"
        assert "wait gave up" in lib.btp_sm100_last_error().decode()
        assert list(detail)[:3] == [1, 0, 0]  # code 1 (timeout), block 0, warp 0
        assert lib.btp_sm100_device_status(stream, detail) == 0  # reported once, then clear
        # the warp that gave up owned (part of) the first sequence; every other sequence is complete and right
        assert O.rel_l2(out[1:].float().cpu(), want[1:]) <= 1e-2
        assert not torch.isfinite(out[0, 0].float()).all()
        # the hook applied to one launch only: the next one is right everywhere and reports nothing
        out, aux = launch()
        assert O.rel_l2(out.float().cpu(), want) <= 1e-2
        if which == "backward":
            assert O.rel_l2(aux.cpu(), dA_w) <= 1e-2
        assert lib.btp_sm100_device_status(stream, detail) == 0
    finally:
        assert lib.btp_sm100_set_wait_limit(previous) == 1_000_000
    assert lib.btp_sm100_set_wait_limit(0) == previous  # 0 restores the default
    _lib.device_status()
