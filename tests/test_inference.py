"""Prefill + decode helpers against golden outputs of the reference's own
spear/nn/phalanx/inference.py (tests/golden/make_golden.py).  The decode step is device-agnostic tensor
code and is checked on CPU; the prefill runs the forward kernel and needs a B200."""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden


def _case(g, L):
    pre = f"L{L}:"
    return {k[len(pre):]: v for k, v in g.items() if k.startswith(pre)}


@pytest.mark.parametrize("L", [40, 64, 7])
def test_decode_steps_match_reference_on_cpu(L):
    from spear_b200.nn.phalanx.inference import JagState, step_jagged

    c = _case(load_golden("inference"), L)
    st = JagState(h_loc=c["h_loc"], r_pref=c["r_pref"], c_prev_loc=c["c_prev_loc"], i=int(c["i"]), block_len=16)
    for j in range(c["Ydec"].shape[-1]):
        t = L + j
        y_t, st = step_jagged(c["A"][..., t], c["X"][..., t], c["C"][..., t], c["V"][..., t], st)
        assert torch.allclose(y_t, c["Ydec"][..., j], rtol=1e-6, atol=1e-6), f"step {j}"
    # the log-space variant of the step agrees with the linear one
    st = JagState(h_loc=c["h_loc"], r_pref=c["r_pref"], c_prev_loc=c["c_prev_loc"], i=int(c["i"]), block_len=16,
                  use_log_r=True, log_r_pref=torch.log(c["r_pref"]))
    for j in range(c["Ydec"].shape[-1]):
        t = L + j
        y_t, st = step_jagged(torch.log(c["A"][..., t]), c["X"][..., t], c["C"][..., t], c["V"][..., t], st, use_log_a=True)
        assert torch.allclose(y_t, c["Ydec"][..., j], rtol=1e-4, atol=1e-4), f"log step {j}"


@pytest.mark.gpu
@pytest.mark.parametrize("L", [40, 64, 7])
def test_prefill_on_the_kernel_then_decode(L):
    from spear_b200.nn.phalanx.inference import parallel_jagged, step_jagged

    c = _case(load_golden("inference"), L)
    dev = lambda t: t.cuda()
    A, X, C, V = (dev(c[k]) for k in "AXCV")
    Y, st = parallel_jagged(A[..., :L], X[..., :L], C[..., :L], V[..., :L], block_len=16)
    rel = lambda got, want: ((got.float().cpu() - want).norm() / want.norm()).item()
    assert Y.shape == c["Y"].shape and rel(Y, c["Y"]) <= 1e-2
    assert st.i == int(c["i"]) and st.block_len == 16
    assert torch.allclose(st.h_loc.cpu(), c["h_loc"], rtol=1e-5, atol=1e-5)
    assert torch.allclose(st.r_pref.cpu(), c["r_pref"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(st.c_prev_loc.cpu(), c["c_prev_loc"], rtol=1e-5, atol=1e-5)
    for j in range(c["Ydec"].shape[-1]):
        t = L + j
        y_t, st = step_jagged(A[..., t], X[..., t], C[..., t], V[..., t], st)
        assert torch.allclose(y_t.cpu(), c["Ydec"][..., j], rtol=1e-5, atol=1e-5), f"step {j}"
    # log-gate prompt through the kernel's log-coefficient entry
    Y2, _ = parallel_jagged(torch.log(A[..., :L]), X[..., :L], C[..., :L], V[..., :L], block_len=16, use_log_a=True)
    assert rel(Y2, c["Y"]) <= 1e-2
    with pytest.raises(NotImplementedError):
        parallel_jagged(A[..., :L], X[..., :L], C[..., :L], V[..., :L], block_len=8)
