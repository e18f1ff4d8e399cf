"""CPU oracle for the streaming form of the block two-pass recurrence (prefill state + decode step).

TEST INFRASTRUCTURE ONLY.  Imported by tests/ as the checker; nothing under spear_b200/ imports it.

Restates, token by token, what the reference's spear/nn/phalanx/inference.py computes:
  * ``step``           - step_jagged (inference.py:177-266), same state fields, plain tensor ops;
  * ``prefill``        - parallel_jagged (inference.py:269-360) as the definition it implements: a block-local
                         scan that restarts every ``block_len`` tokens, a one-hop carry from the previous block's
                         last local value scaled by the running gate product, then ``y * C + V``; and the
                         hand-off state of inference.py:333-358, including its behaviour when the prompt ends on
                         a block boundary (h_loc keeps the finished block's last value).
Pinned to outputs of the reference itself: tests/golden/inference.npz (made by tests/golden/make_golden.py).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class OracleState:
    h_loc: torch.Tensor
    r_pref: torch.Tensor | None
    c_prev_loc: torch.Tensor
    i: int
    block_len: int
    use_log_r: bool = False
    log_r_pref: torch.Tensor | None = None


def step(A_t, X_t, C_t, V_t, st: OracleState, *, use_log_a: bool = False):
    """inference.py:199-266."""
    a = A_t.exp() if use_log_a else A_t
    h = a.unsqueeze(-1) * st.h_loc + X_t
    log_space = st.use_log_r or use_log_a
    if log_space:
        prev = st.log_r_pref if st.log_r_pref is not None else torch.zeros_like(a)
        log_r = prev + torch.log(a.clamp_min(torch.finfo(a.dtype).tiny))
        r = torch.exp(log_r)
    else:
        prev = st.r_pref if st.r_pref is not None else torch.ones_like(a)
        r = a * prev
        log_r = None
    y = (h + r.unsqueeze(-1) * st.c_prev_loc) * C_t + V_t
    if st.i + 1 == st.block_len:
        return y, OracleState(torch.zeros_like(h), None if log_space else torch.ones_like(A_t), h.clone(), 0,
                              st.block_len, log_space, torch.zeros_like(A_t) if log_space else None)
    return y, OracleState(h, None if log_space else r, st.c_prev_loc, st.i + 1, st.block_len, log_space,
                          log_r if log_space else None)


def prefill(A, X, C, V, *, block_len: int = 16, use_log_a: bool = False):
    """Sequential definition of inference.py:269-360.  A (B,H,L), X/C/V (B,H,D,L); returns (Y, OracleState)."""
    a = (A.exp() if use_log_a else A).to(torch.float64)
    x = X.to(torch.float64)
    Bsz, H, D, L = x.shape
    h = torch.zeros(Bsz, H, D, dtype=torch.float64)
    r = torch.ones(Bsz, H, dtype=torch.float64)
    c_prev = torch.zeros(Bsz, H, D, dtype=torch.float64)
    ys = []
    h_last = h
    r_last = r
    c_prev_last_complete = c_prev
    for t in range(L):
        i = t % block_len
        if i == 0:
            if t > 0:
                c_prev = h
                c_prev_last_complete = h
            h = torch.zeros_like(h)
            r = torch.ones_like(r)
        h = a[..., t].unsqueeze(-1) * h + x[..., t]
        r = r * a[..., t]
        ys.append(h + r.unsqueeze(-1) * c_prev)
        h_last, r_last = h, r
    Y = torch.stack(ys, dim=-1) * C.to(torch.float64) + V.to(torch.float64)
    tail_i = (L - 1) % block_len
    if tail_i == block_len - 1:  # inference.py:339-342
        c_tail, r_tail, i_next = h_last.clone(), torch.ones_like(r_last), 0
    else:                        # inference.py:343-350
        c_tail = c_prev_last_complete if L // block_len > 0 else torch.zeros_like(h_last)
        r_tail, i_next = r_last, tail_i + 1
    st = OracleState(h_last.to(V.dtype), r_tail.to(A.dtype if not use_log_a else torch.float32), c_tail.to(V.dtype),
                     i_next, block_len)
    return Y.to(V.dtype), st
