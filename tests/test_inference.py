"""Prefill + decode against golden outputs of the reference's own spear/nn/phalanx/inference.py
(tests/golden/make_golden.py).  On CPU the oracle restatement is pinned to those outputs; on the GPU the
kernels (forward kernel for the prompt, one launch for the hand-off state, one launch per decode step)
are checked against the golden outputs and against the oracle on larger random cases."""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden

LENGTHS = [40, 64, 7]


def _case(g, L):
    pre = f"L{L}:"
    return {k[len(pre):]: v for k, v in g.items() if k.startswith(pre)}


# ------------------------------------------------------------------ CPU: the oracle against the reference's outputs
@pytest.mark.parametrize("L", LENGTHS)
def test_oracle_step_matches_reference(L):
    import jagged_oracle as O

    c = _case(load_golden("inference"), L)
    st = O.OracleState(c["h_loc"], c["r_pref"], c["c_prev_loc"], int(c["i"]), 16)
    for j in range(c["Ydec"].shape[-1]):
        t = L + j
        y_t, st = O.step(c["A"][..., t], c["X"][..., t], c["C"][..., t], c["V"][..., t], st)
        assert torch.allclose(y_t, c["Ydec"][..., j], rtol=1e-6, atol=1e-6), f"step {j}"
    st = O.OracleState(c["h_loc"], c["r_pref"], c["c_prev_loc"], int(c["i"]), 16, True, torch.log(c["r_pref"]))
    for j in range(c["Ydec"].shape[-1]):
        t = L + j
        y_t, st = O.step(torch.log(c["A"][..., t]), c["X"][..., t], c["C"][..., t], c["V"][..., t], st, use_log_a=True)
        assert torch.allclose(y_t, c["Ydec"][..., j], rtol=1e-4, atol=1e-4), f"log step {j}"


@pytest.mark.parametrize("L", LENGTHS)
def test_oracle_prefill_matches_reference(L):
    import jagged_oracle as O

    c = _case(load_golden("inference"), L)
    Y, st = O.prefill(c["A"][..., :L], c["X"][..., :L], c["C"][..., :L], c["V"][..., :L])
    assert torch.allclose(Y, c["Y"], rtol=1e-5, atol=1e-5)
    assert st.i == int(c["i"])
    assert torch.allclose(st.h_loc, c["h_loc"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(st.r_pref, c["r_pref"], rtol=1e-5, atol=1e-7)
    assert torch.allclose(st.c_prev_loc, c["c_prev_loc"], rtol=1e-5, atol=1e-6)
    Ylog, _ = O.prefill(torch.log(c["A"][..., :L]), c["X"][..., :L], c["C"][..., :L], c["V"][..., :L], use_log_a=True)
    assert torch.allclose(Ylog, c["Y"], rtol=1e-4, atol=1e-4)


def test_streaming_helpers_have_no_cpu_path():
    from spear_b200.nn.phalanx.inference import JagState, parallel_jagged, step_jagged

    A, X = torch.rand(1, 2, 16), torch.randn(1, 2, 16, 16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        parallel_jagged(A, X, X, X, block_len=16)
    st = JagState(h_loc=X[..., 0], r_pref=A[..., 0], c_prev_loc=X[..., 0], i=1, block_len=16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        step_jagged(A[..., 0], X[..., 0], X[..., 0], X[..., 0], st)


# ------------------------------------------------------------------ GPU: the kernels
@pytest.mark.gpu
@pytest.mark.parametrize("L", LENGTHS)
def test_prefill_on_the_kernel_then_decode(L):
    from spear_b200 import _lib
    from spear_b200.nn.phalanx.inference import parallel_jagged, step_jagged

    c = _case(load_golden("inference"), L)
    dev = lambda t: t.cuda()
    A, X, C, V = (dev(c[k]) for k in "AXCV")
    n0 = _lib.launch_count()
    Y, st = parallel_jagged(A[..., :L], X[..., :L], C[..., :L], V[..., :L], block_len=16)
    # the fixture's prompt is float32: two launches of the forward kernel (X as two bf16 terms) + the state kernel
    assert A.dtype == torch.float32 and _lib.launch_count() - n0 == 3
    rel = lambda got, want: ((got.float().cpu() - want).norm() / want.norm()).item()
    # Y at the accuracy of a float32 evaluation (the reference computes Y in the input type, inference.py:269-360)
    assert Y.shape == c["Y"].shape and rel(Y, c["Y"]) <= 2e-5
    assert torch.allclose(Y.cpu(), c["Y"], rtol=1e-4, atol=1e-4)
    # the same prompt in bf16: one launch of the forward kernel, bf16 accuracy
    n0 = _lib.launch_count()
    Yb, _ = parallel_jagged(*(t[..., :L].bfloat16() for t in (A, X, C, V)), block_len=16)
    assert _lib.launch_count() - n0 == 2 and Yb.dtype == torch.bfloat16 and rel(Yb, c["Y"]) <= 2e-2
    assert st.i == int(c["i"]) and st.block_len == 16
    assert torch.allclose(st.h_loc.cpu(), c["h_loc"], rtol=1e-5, atol=1e-5)
    assert torch.allclose(st.r_pref.cpu(), c["r_pref"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(st.c_prev_loc.cpu(), c["c_prev_loc"], rtol=1e-5, atol=1e-5)
    st0 = st
    for j in range(c["Ydec"].shape[-1]):
        t = L + j
        n0 = _lib.launch_count()
        y_t, st = step_jagged(A[..., t], X[..., t], C[..., t], V[..., t], st)
        assert _lib.launch_count() - n0 == 1
        assert torch.allclose(y_t.cpu(), c["Ydec"][..., j], rtol=1e-5, atol=1e-5), f"step {j}"
    # the state that went in is still valid: stepping from it again gives the same first output
    y_again, _ = step_jagged(A[..., L], X[..., L], C[..., L], V[..., L], st0)
    assert torch.allclose(y_again.cpu(), c["Ydec"][..., 0], rtol=1e-5, atol=1e-5)
    # log-gate prompt through the kernel's log-coefficient entry, then log-space decode
    Y2, st2 = parallel_jagged(torch.log(A[..., :L]), X[..., :L], C[..., :L], V[..., :L], block_len=16, use_log_a=True)
    assert rel(Y2, c["Y"]) <= 2e-5
    assert torch.allclose(st2.r_pref.cpu(), c["r_pref"], rtol=1e-4, atol=1e-6)
    st2.use_log_r, st2.log_r_pref, st2.r_pref = True, torch.log(st2.r_pref), None
    for j in range(c["Ydec"].shape[-1]):
        t = L + j
        y_t, st2 = step_jagged(torch.log(A[..., t]), X[..., t], C[..., t], V[..., t], st2, use_log_a=True)
        assert st2.use_log_r and st2.r_pref is None
        assert torch.allclose(y_t.cpu(), c["Ydec"][..., j], rtol=1e-4, atol=1e-4), f"log step {j}"
    with pytest.raises(NotImplementedError):
        parallel_jagged(A[..., :L], X[..., :L], C[..., :L], V[..., :L], block_len=8)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("L", [1, 16, 33, 96, 250])
def test_streaming_kernels_against_oracle(L, dtype):
    """Random prompts of awkward lengths, then 40 decode steps, in both storage types."""
    import jagged_oracle as O
    from spear_b200.nn.phalanx.inference import parallel_jagged, step_jagged

    g = torch.Generator().manual_seed(1000 + L)
    B, H, D, steps = 3, 5, 16, 40
    total = L + steps
    A = torch.sigmoid(torch.randn(B, H, total, generator=g) + 2.0).to(dtype)
    X, C, V = (torch.randn(B, H, D, total, generator=g).mul(0.5).to(dtype) for _ in range(3))
    # oracle in float32 on the same (already rounded) inputs
    Af, Xf, Cf, Vf = (t.float() for t in (A, X, C, V))
    Yo, so = O.prefill(Af[..., :L], Xf[..., :L], Cf[..., :L], Vf[..., :L])
    Ad, Xd, Cd, Vd = (t.cuda() for t in (A, X, C, V))
    Y, st = parallel_jagged(Ad[..., :L], Xd[..., :L], Cd[..., :L], Vd[..., :L], block_len=16)
    assert Y.dtype == dtype and st.h_loc.dtype == dtype and st.r_pref.dtype == dtype
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    assert torch.allclose(Y.float().cpu(), Yo, **tol)
    stol = dict(rtol=1e-2, atol=1e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    assert st.i == so.i
    assert torch.allclose(st.h_loc.float().cpu(), so.h_loc, **stol)
    assert torch.allclose(st.r_pref.float().cpu(), so.r_pref, **stol)
    assert torch.allclose(st.c_prev_loc.float().cpu(), so.c_prev_loc, **stol)
    # decode: feed the oracle the kernel's own (rounded) state each step so that one step's rounding is what is compared
    for j in range(steps):
        t = L + j
        so = O.OracleState(st.h_loc.float().cpu(), st.r_pref.float().cpu(), st.c_prev_loc.float().cpu(), st.i, 16)
        yo, so_next = O.step(Af[..., t], Xf[..., t], Cf[..., t], Vf[..., t], so)
        y_t, st = step_jagged(Ad[..., t], Xd[..., t], Cd[..., t], Vd[..., t], st)
        assert y_t.dtype == dtype and st.i == so_next.i
        assert torch.allclose(y_t.float().cpu(), yo, **stol), f"step {j}"
        assert torch.allclose(st.h_loc.float().cpu(), so_next.h_loc, **stol)
        assert torch.allclose(st.r_pref.float().cpu(), so_next.r_pref, **stol)
        assert torch.allclose(st.c_prev_loc.float().cpu(), so_next.c_prev_loc, **stol)


@pytest.mark.gpu
def test_decode_step_c_abi_argument_errors():
    from spear_b200 import _btp

    x = torch.zeros(4, 16, device="cuda")
    a = torch.ones(4, device="cuda")
    ok = dict(block_complete=False, gate_is_log=False, r_is_log=False)
    with pytest.raises(RuntimeError, match="share shape and dtype"):
        _btp.decode_step(a, x, x.bfloat16(), x, x.clone(), x, a, x, x.clone(), a.clone(), None, **ok)
    with pytest.raises(RuntimeError, match="completes a block"):
        _btp.decode_step(a, x, x, x, x.clone(), x, a, x, x.clone(), a.clone(), None,
                         block_complete=True, gate_is_log=False, r_is_log=False)
    with pytest.raises(RuntimeError, match="bfloat16 or float32"):
        h = x.half()
        _btp.decode_step(a, h, h, h, h.clone(), h, a, h, h.clone(), a.clone(), None, **ok)
