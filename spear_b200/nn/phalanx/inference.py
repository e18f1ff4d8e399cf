"""Prefill and per-token decode for the Phalanx sliding-window recurrence on the sm_100a kernel.

Mirror of the reference's streaming helpers (spear/nn/phalanx/inference.py:142-360): the same ``JagState``
fields, ``parallel_jagged`` (prompt prefill returning the outputs and the hand-off state) and
``step_jagged`` (one decode step).  The reference runs two nested Python loops over blocks and tokens for
the prefill; here the prompt goes through the BTP forward kernel in one launch, the hand-off state (which
depends on at most the last 32 tokens) comes from one small kernel, and a decode step is one kernel launch
instead of a dozen tensor ops.  CUDA tensors only - there is no CPU path; block_len must be 16.
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


_KERNEL_DTYPES = (torch.bfloat16, torch.float32)


def _kernel_dtype(*tensors):
    """Storage type the kernels run in: the promoted type if it is bfloat16 or float32, else float32."""
    dt = tensors[0].dtype
    for t in tensors[1:]:
        if t.dtype != dt:
            dt = torch.promote_types(dt, t.dtype)
    return dt, (dt if dt in _KERNEL_DTYPES else torch.float32)


def _as(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return t if (t.dtype == dtype and t.is_contiguous()) else t.to(dtype).contiguous()


@torch.no_grad()
def parallel_jagged(A, X, C, V, *, block_len: int, use_log_a: bool = False):
    """Prompt prefill (signature of inference.py:269-279): returns (Y [B,H,D,L], JagState).

    A: (B,H,L) gates (log gates if use_log_a), X: (B,H,D,L) driving term, C, V: (B,H,D,L).
    Any L >= 1: the prompt is padded to a multiple of 16 with neutral tokens exactly as the reference pads it.
    bf16 prompts take one launch of the forward kernel; wider prompts take two (see below) and keep their accuracy.
    A kernel wait that gives up leaves its part of Y unwritten and is reported by `_lib.device_status()`: poll it
    at a synchronisation point the caller already has (once per request or per step).
    """
    if block_len != BLOCK:
        raise NotImplementedError(f"the kernel's block length is {BLOCK} (got block_len={block_len})")
    if not (X.is_cuda and A.is_cuda):
        raise RuntimeError("parallel_jagged needs CUDA tensors: this package has no CPU path")
    Bsz, H, D, L = V.shape
    if D != 16:
        raise ValueError("head_dim must be 16")
    if L < 1:
        raise ValueError("the prompt must hold at least one token")
    pad = (-L) % BLOCK
    # The kernel takes bf16 x and bf16 / float32 gates (float32 log gates); tensors already in that form are
    # passed as they are, without a copy.
    coeff = A.float() if (use_log_a or A.dtype not in _KERNEL_DTYPES) else A
    # A prompt wider than bf16 (float32, float16) is fed as TWO bf16 terms, X = hi + lo: the op is linear in x, so
    # btp(a, hi) + btp(a, lo) is the result for X itself to about 2^-17, at the price of a second launch.  Y then
    # has the accuracy of the input type, as in the reference, and agrees with the hand-off state below, which
    # is computed from the unrounded X.
    terms = [X if X.dtype == torch.bfloat16 else X.to(torch.bfloat16)]
    if X.dtype != torch.bfloat16:
        terms.append((X.float() - terms[0].float()).to(torch.bfloat16))
    if pad:
        coeff = torch.nn.functional.pad(coeff, (0, pad), value=0.0 if use_log_a else 1.0)
        terms = [torch.nn.functional.pad(t, (0, pad), value=0.0) for t in terms]
    coeff = coeff.contiguous()
    low = len(terms) == 1 and V.dtype == torch.bfloat16 and C.dtype == torch.bfloat16
    y = None
    for t in terms:
        t = t.contiguous()
        yt = torch.empty(t.shape, device=t.device, dtype=torch.bfloat16 if low else torch.float32)
        _native.forward(coeff, t, yt, None, 2, 32, log_coeff=use_log_a)
        y = yt if y is None else y.add_(yt)
    y = y[..., :L] if pad else y
    if low:
        Y = torch.addcmul(V, y, C)  # one pass, fp32 arithmetic inside, one rounding
    else:
        Y = torch.addcmul(V.float(), y, C.float()).to(V.dtype)

    # hand-off state (inference.py:333-358): one launch over the last partial block and the complete one before it
    _, xdt = _kernel_dtype(X)
    _, adt = _kernel_dtype(A)
    h_tail = torch.empty((Bsz, H, D), device=X.device, dtype=xdt)
    c_prev_tail = torch.empty_like(h_tail)
    r_tail = torch.empty((Bsz, H), device=X.device, dtype=adt)
    _native.prefill_state(_as(A, adt), _as(X, xdt), h_tail, r_tail, c_prev_tail, gate_is_log=use_log_a)
    state = JagState(h_loc=h_tail.to(V.dtype), r_pref=r_tail.to(A.dtype), c_prev_loc=c_prev_tail.to(V.dtype),
                     i=(L % BLOCK), block_len=block_len, use_log_r=False, log_r_pref=None)
    return Y, state


@torch.no_grad()
def step_jagged(A_t, X_t, C_t, V_t, state: JagState, *, use_log_a: bool = False):
    """One decode step (inference.py:177-266): returns (y_t [B,H,D], new JagState).

    One kernel launch.  Like the reference it returns fresh state tensors and leaves `state` valid; the frozen
    `c_prev_loc` is shared between consecutive states until a block completes.  Arithmetic is fp32 with a single
    rounding to the storage type, where the reference rounds after every tensor op.
    """
    if not (A_t.is_cuda and X_t.is_cuda and state.h_loc.is_cuda):
        raise RuntimeError("step_jagged needs CUDA tensors: this package has no CPU path")
    if X_t.shape[-1] != 16 or A_t.shape != X_t.shape[:-1] or not (
            C_t.shape == V_t.shape == X_t.shape == state.h_loc.shape == state.c_prev_loc.shape):
        raise ValueError("step_jagged takes A_t [B,H] and X_t, C_t, V_t, state.h_loc, state.c_prev_loc [B,H,16]")
    if state.block_len != BLOCK:
        raise NotImplementedError(f"the kernel's block length is {BLOCK} (got block_len={state.block_len})")
    log_space = bool(state.use_log_r or use_log_a)
    r_prev = state.log_r_pref if log_space else state.r_pref
    out_dt, dt = _kernel_dtype(X_t, C_t, V_t, state.h_loc, state.c_prev_loc)
    gate_out_dt, gdt = _kernel_dtype(*((A_t,) if r_prev is None else (A_t, r_prev)))
    a_t, x_t, c_t, v_t = _as(A_t, gdt), _as(X_t, dt), _as(C_t, dt), _as(V_t, dt)
    h_in, cp_in = _as(state.h_loc, dt), _as(state.c_prev_loc, dt)
    r_in = None if r_prev is None else _as(r_prev, gdt)
    done = state.i + 1 == state.block_len
    if r_in is not None and r_in.shape != a_t.shape:
        raise ValueError("the state's gate product must have the shape of A_t")
    buf = torch.empty((3 if done else 2,) + x_t.shape, device=x_t.device, dtype=dt)  # one allocation
    y_t, h_out = buf[0], buf[1]
    cp_out = buf[2] if done else None
    r_out = torch.empty_like(a_t)
    _native.decode_step(a_t, x_t, c_t, v_t, y_t, h_in, r_in, cp_in, h_out, r_out, cp_out,
                        block_complete=done, gate_is_log=use_log_a, r_is_log=log_space, _checked=True)
    if dt != out_dt:
        y_t, h_out = y_t.to(out_dt), h_out.to(out_dt)
        cp_out = None if cp_out is None else cp_out.to(out_dt)
    if gdt != gate_out_dt:
        r_out = r_out.to(gate_out_dt)
    return y_t, JagState(h_loc=h_out, r_pref=None if log_space else r_out,
                         c_prev_loc=cp_out if done else state.c_prev_loc, i=0 if done else state.i + 1,
                         block_len=state.block_len, use_log_r=log_space, log_r_pref=r_out if log_space else None)
