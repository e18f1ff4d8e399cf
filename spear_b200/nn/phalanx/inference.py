"""Prefill and per-token decode for the Phalanx sliding-window recurrence on the sm_100a kernel.

Mirror of the reference's streaming helpers (spear/nn/phalanx/inference.py:142-360): the same ``JagState``
fields, ``parallel_jagged`` (prompt prefill returning the outputs and the hand-off state) and
``step_jagged`` (one decode step).  The reference runs two nested Python loops over blocks and tokens for
the prefill; here the prompt goes through the BTP forward kernel in one launch and only the hand-off state,
which depends on at most the last 32 tokens, is formed with a few small tensor ops.  The decode step is a
handful of elementwise device ops on [B, H, 16] tensors.  CUDA tensors only; block_len must be 16.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ... import _btp as _native

__all__ = ["JagState", "parallel_jagged", "step_jagged"]

BLOCK = 16


@dataclass
class JagState:
    """Streaming state, field for field the reference's (inference.py:142-174)."""

    h_loc: torch.Tensor            # (B, H, D) block-local accumulator
    r_pref: torch.Tensor | None    # (B, H) inclusive product of the gates inside the current block
    c_prev_loc: torch.Tensor       # (B, H, D) frozen last local value of the previous block
    i: int                         # in-block index of the next token
    block_len: int
    use_log_r: bool = False
    log_r_pref: torch.Tensor | None = None

    def clone_detached(self) -> "JagState":
        return JagState(
            h_loc=self.h_loc.clone(),
            r_pref=None if self.r_pref is None else self.r_pref.clone(),
            c_prev_loc=self.c_prev_loc.clone(),
            i=int(self.i),
            block_len=int(self.block_len),
            use_log_r=bool(self.use_log_r),
            log_r_pref=None if self.log_r_pref is None else self.log_r_pref.clone(),
        )


def _local_tail(a_blk: torch.Tensor, x_blk: torch.Tensor):
    """Zero-initialised scan over one (possibly partial) block: last local value (B,H,D) and gate product (B,H)."""
    h = torch.zeros(x_blk.shape[:-1], dtype=torch.float32, device=x_blk.device)
    r = torch.ones(a_blk.shape[:-1], dtype=torch.float32, device=a_blk.device)
    for k in range(a_blk.shape[-1]):  # at most 16 steps on [B,H,D] tensors
        ak = a_blk[..., k].float()
        h = ak.unsqueeze(-1) * h + x_blk[..., k].float()
        r = r * ak
    return h, r


@torch.no_grad()
def parallel_jagged(A, X, C, V, *, block_len: int, use_log_a: bool = False):
    """Prompt prefill (signature of inference.py:269-279): returns (Y [B,H,D,L], JagState).

    A: (B,H,L) gates (log gates if use_log_a), X: (B,H,D,L) driving term, C, V: (B,H,D,L).
    Any L >= 1: the prompt is padded to a multiple of 16 with neutral tokens exactly as the reference pads it.
    """
    if block_len != BLOCK:
        raise NotImplementedError(f"the kernel's block length is {BLOCK} (got block_len={block_len})")
    if not (X.is_cuda and A.is_cuda):
        raise RuntimeError("parallel_jagged needs CUDA tensors: this package has no CPU path")
    Bsz, H, D, L = V.shape
    if D != 16:
        raise ValueError("head_dim must be 16")
    pad = (-L) % BLOCK
    a_lin = A.float().exp() if use_log_a else A.float()
    coeff = A.float() if use_log_a else a_lin
    x = X.to(torch.bfloat16)
    if pad:
        coeff = torch.nn.functional.pad(coeff, (0, pad), value=0.0 if use_log_a else 1.0)
        x = torch.nn.functional.pad(x, (0, pad), value=0.0)
    coeff = coeff.contiguous()
    x = x.contiguous()
    y = torch.empty(x.shape, device=x.device, dtype=torch.float32)
    _native.forward(coeff, x, y, None, 2, 32, log_coeff=use_log_a)
    Y = (y[..., :L] * C.float() + V.float()).to(V.dtype)

    # hand-off state (inference.py:333-358): it depends on the last partial block and the last complete one
    n_completed = L // BLOCK
    tail_i = (L - 1) % BLOCK
    s_last = (L - 1) // BLOCK * BLOCK
    h_tail, r_tail = _local_tail(a_lin[..., s_last:L], X[..., s_last:L])
    if tail_i == BLOCK - 1:
        c_prev_tail = h_tail.clone()
        r_tail = torch.ones_like(r_tail)
        i_next = 0
    else:
        if n_completed > 0:
            c_prev_tail, _ = _local_tail(a_lin[..., s_last - BLOCK:s_last], X[..., s_last - BLOCK:s_last])
        else:
            c_prev_tail = torch.zeros_like(h_tail)
        i_next = tail_i + 1
    state = JagState(h_loc=h_tail.to(V.dtype), r_pref=r_tail.to(a_lin.dtype if A.dtype == torch.float32 else A.dtype),
                     c_prev_loc=c_prev_tail.to(V.dtype), i=i_next, block_len=block_len, use_log_r=False, log_r_pref=None)
    return Y, state


@torch.no_grad()
def step_jagged(A_t, X_t, C_t, V_t, state: JagState, *, use_log_a: bool = False):
    """One decode step (inference.py:177-266): returns (y_t [B,H,D], new JagState)."""
    a_t = A_t.exp() if use_log_a else A_t
    h_loc = a_t.unsqueeze(-1) * state.h_loc + X_t
    log_space = state.use_log_r or use_log_a
    if log_space:
        tiny = torch.finfo(a_t.dtype).tiny
        prev = state.log_r_pref if state.log_r_pref is not None else torch.zeros_like(a_t)
        log_r = prev + torch.log(a_t.clamp_min(tiny))
        r_pref = torch.exp(log_r)
    else:
        prev = state.r_pref if state.r_pref is not None else torch.ones_like(a_t)
        r_pref = a_t * prev
        log_r = None
    y_t = (h_loc + r_pref.unsqueeze(-1) * state.c_prev_loc) * C_t + V_t
    i_next = state.i + 1
    if i_next == state.block_len:  # block complete: freeze its last local value, start the next block empty
        return y_t, JagState(h_loc=torch.zeros_like(h_loc), r_pref=None if log_space else torch.ones_like(A_t),
                             c_prev_loc=h_loc.clone(), i=0, block_len=state.block_len, use_log_r=log_space,
                             log_r_pref=torch.zeros_like(A_t) if log_space else None)
    return y_t, JagState(h_loc=h_loc, r_pref=None if log_space else r_pref, c_prev_loc=state.c_prev_loc, i=i_next,
                         block_len=state.block_len, use_log_r=log_space, log_r_pref=log_r if log_space else None)
