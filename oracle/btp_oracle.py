"""CPU oracle for the block two-pass (BTP) sliding-window recurrence.

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA path is
compared with.  Nothing in the shipped package imports it; only the tests, the
smoke check and the CPU-baseline leg of the benchmark do.

It restates, in plain torch CPU ops, the algorithm of the reference's PyTorch
path (spear/ops/btp/reference.py):

* ``lmat_log_stable``   follows ``segsum_stable`` + ``construct_L_exp_segsum_log_stable``
  (reference.py:38-52): row-wise cumulative sums of log a inside the lower
  triangle, never a difference of two long prefixes.
* ``lmat_product``      follows ``construct_L_ref`` (reference.py:55-77): explicit
  products in float64.
* ``lmat_cumprod``      follows ``construct_L_masked_cumprod`` (reference.py:79-90):
  masked column-wise cumulative product in linear space (safe for a == 0).
* ``btp_forward``       follows ``block_two_pass`` (reference.py:105-139): local
  pass per 16-token block, then ONE hop of carry from the block-local last
  token of the previous block, scaled by a_0 * L[:, 0].
* ``btp_backward``      closed form of the gradient of ``btp_forward`` (what
  autograd of reference.py:105-139 yields; the reference kernel's version is
  csrc/btp/btp-backwards.cu:337-413,466-608,637-797), written without any
  division by a so that a == 0 and a == 1 need no special cases.

Parity pin: tests/golden/*.npz hold inputs and outputs produced by importing
the reference's own reference.py (script tests/golden/make_golden.py); the CPU
test-suite checks every function here against them.
"""

from __future__ import annotations

import torch

BLOCK = 16  # tokens per block (spear/ops/btp/interface.py:24)
HEAD_DIM = 16  # channels per head (spear/ops/btp/interface.py:23)

__all__ = [
    "BLOCK",
    "HEAD_DIM",
    "lmat_log_stable",
    "lmat_product",
    "lmat_cumprod",
    "btp_forward",
    "btp_backward",
    "btp_forward_backward_autograd",
    "rel_l2",
    "error_metrics",
]


def _blocks(t: torch.Tensor, block: int) -> torch.Tensor:
    """[..., L] -> [..., L/block, block] (reference.py:119 rearrange)."""
    if t.shape[-1] % block != 0:
        raise ValueError(f"length {t.shape[-1]} is not a multiple of {block}")
    return t.reshape(*t.shape[:-1], t.shape[-1] // block, block)


def lmat_log_stable(a_blk: torch.Tensor) -> torch.Tensor:
    """L[..., r, c] = exp(sum_{j=c+1..r} log a_j) for r >= c, else 0.

    a_blk: [..., n] coefficients of one block.  The sum is accumulated row by
    row over a matrix whose entry (j, c) is log a_j when j > c and 0 otherwise,
    which is the summation order of reference.py:38-52.
    """
    n = a_blk.shape[-1]
    la = torch.log(a_blk)
    j = torch.arange(n).unsqueeze(-1)
    c = torch.arange(n).unsqueeze(0)
    terms = torch.where(j > c, la.unsqueeze(-1), torch.zeros((), dtype=la.dtype))
    seg = torch.cumsum(terms, dim=-2)
    seg = torch.where(j >= c, seg, torch.full((), float("-inf"), dtype=la.dtype))
    return torch.exp(seg)


def lmat_product(a_blk: torch.Tensor) -> torch.Tensor:
    """Explicit products in float64 (reference.py:55-77); result in a's dtype."""
    n = a_blk.shape[-1]
    a64 = a_blk.double()
    one = torch.ones_like(a64[..., 0])
    zero = torch.zeros_like(one)
    rows = []
    for r in range(n):
        row = [zero] * n
        row[r] = one
        for c in range(r - 1, -1, -1):
            row[c] = row[c + 1] * a64[..., c + 1]
        rows.append(torch.stack(row, dim=-1))
    return torch.stack(rows, dim=-2).to(a_blk.dtype)


def lmat_cumprod(a_blk: torch.Tensor) -> torch.Tensor:
    """Masked column-wise cumulative product in linear space (reference.py:79-90)."""
    n = a_blk.shape[-1]
    j = torch.arange(n).unsqueeze(-1)
    c = torch.arange(n).unsqueeze(0)
    factors = torch.where(j > c, a_blk.unsqueeze(-1), torch.ones((), dtype=a_blk.dtype))
    prod = torch.cumprod(factors, dim=-2)
    return torch.where(j >= c, prod, torch.zeros((), dtype=a_blk.dtype))


_LMAT = {"log": lmat_log_stable, "product": lmat_product, "cumprod": lmat_cumprod}


def _local_and_scale(a: torch.Tensor, x: torch.Tensor, lmat: str, block: int):
    """Returns L [B,H,NB,r,c], local pass v [B,H,D,NB,r], carry scale P [B,H,NB,r]."""
    ab = _blocks(a, block)
    xb = _blocks(x, block)
    L = _LMAT[lmat](ab)
    v = torch.einsum("bhnrc,bhdnc->bhdnr", L, xb)  # reference.py:124-125
    P = ab[..., 0:1] * L[..., :, 0]  # reference.py:129-132: a_0 * first column
    return L, v, P


def btp_forward(a: torch.Tensor, x: torch.Tensor, k: int = 2, lmat: str = "log", block: int = BLOCK) -> torch.Tensor:
    """y[B,H,D,L] of the block two-pass op (reference.py:105-139).

    a: [B,H,L] linear-space coefficients, x: [B,H,D,L]; same float dtype.
    k=2 adds the one-hop carry; k=1 is the local pass alone (the kernel's
    k==1 mode, csrc/btp/btp-forward.cu:276).
    """
    if a.dim() != 3 or x.dim() != 4 or a.shape[:2] != x.shape[:2] or a.shape[-1] != x.shape[-1]:
        raise ValueError(f"shape mismatch: a {tuple(a.shape)} x {tuple(x.shape)}")
    if k not in (1, 2):
        raise ValueError("k must be 1 or 2")
    _, v, P = _local_and_scale(a, x, lmat, block)
    y = v.clone()
    if k == 2 and v.shape[3] > 1:
        carry = v[:, :, :, :-1, -1]  # block-local last token of the previous block
        y[:, :, :, 1:, :] += P[:, :, None, 1:, :] * carry[..., None]  # reference.py:133-136
    return y.reshape(x.shape)


def btp_backward(
    a: torch.Tensor,
    x: torch.Tensor,
    dy: torch.Tensor,
    k: int = 2,
    lmat: str = "log",
    block: int = BLOCK,
):
    """(dA[B,H,L], dx[B,H,D,L]) for upstream gradient dy, closed form.

    With gw = dy . L (raw dy), dCarry_{i+1}[d] = sum_r dy_{i+1}[d,r] P_{i+1}[r]:
      dx_i[d,c] = gw_i[d,c] + L_i[15,c] * dCarry_{i+1}[d]
      dA_i[t]   = sum_d ( gw_i[d,t] * y_i[d,t-1] + dCarry_{i+1}[d] * L_i[15,t] * v_i[d,t-1] )
    where y_i[:, -1] is the carry into block i and v_i[:, -1] = 0.
    """
    L, v, P = _local_and_scale(a, x, lmat, block)
    dyb = _blocks(dy.to(a.dtype), block)
    nb = v.shape[3]
    gw = torch.einsum("bhdnr,bhnrc->bhdnc", dyb, L)
    carry = torch.zeros_like(v[..., 0])  # [B,H,D,NB]
    dcarry_in = torch.zeros_like(carry)
    if k == 2 and nb > 1:
        carry[..., 1:] = v[:, :, :, :-1, -1]
        dcarry = torch.einsum("bhdnr,bhnr->bhdn", dyb, P)
        dcarry_in[..., :-1] = dcarry[..., 1:]
    y = v + P[:, :, None] * carry[..., None]
    lrow = L[..., -1, :]  # [B,H,NB,c]
    dx = gw + lrow[:, :, None] * dcarry_in[..., None]
    y_prev = torch.cat([carry[..., None], y[..., :-1]], dim=-1)
    v_prev = torch.cat([torch.zeros_like(carry[..., None]), v[..., :-1]], dim=-1)
    dA = (gw * y_prev + dcarry_in[..., None] * lrow[:, :, None] * v_prev).sum(dim=2)
    return dA.reshape(a.shape), dx.reshape(x.shape)


def btp_forward_backward_autograd(a: torch.Tensor, x: torch.Tensor, dy: torch.Tensor, lmat: str = "log"):
    """Forward + autograd backward, the way the reference's CPU path is used
    (spear/ops/btp/runners.py:151-163).  This is what the CPU baseline times."""
    a = a.detach().clone().requires_grad_(True)
    x = x.detach().clone().requires_grad_(True)
    y = btp_forward(a, x, 2, lmat)
    y.backward(dy.to(y.dtype))
    return y.detach(), a.grad, x.grad


def rel_l2(got: torch.Tensor, want: torch.Tensor) -> float:
    """||got - want||_2 / ||want||_2 in float64."""
    g = got.detach().double().flatten().cpu()
    w = want.detach().double().flatten().cpu()
    den = torch.linalg.vector_norm(w).item()
    num = torch.linalg.vector_norm(g - w).item()
    return num / den if den > 0 else num


def error_metrics(got: torch.Tensor, want: torch.Tensor, eps: float = 1e-7) -> dict:
    """max/mean abs, max/mean rel, rmse (spear/testing/numerics/metrics.py:25-44) + rel_l2."""
    g = got.detach().float().cpu()
    w = want.detach().float().cpu()
    ad = (g - w).abs()
    rd = ad / (w.abs() + eps)
    return {
        "max_abs": ad.max().item(),
        "mean_abs": ad.mean().item(),
        "max_rel": rd.max().item(),
        "mean_rel": rd.mean().item(),
        "rmse": ad.square().mean().sqrt().item(),
        "rel_l2": rel_l2(got, want),
    }


def phalanx_forward(state: dict, u: torch.Tensor, k: int = 2, kv_heads: int | None = None,
                    decay_dtype: torch.dtype | None = None) -> torch.Tensor:
    """The Phalanx layer's data flow around the oracle op, in the dtype of `u` on CPU.

    `decay_dtype`: the reference layer computes its projections and the sigmoid in bfloat16
    (spear/nn/phalanx/swr.py:146,170,216): the logits of the decay are bfloat16 numbers, the decay it hands to
    the op is one, and autograd differentiates the sigmoid at that rounded value, a(1 - a).  Decays close to one
    (0.9995) do not survive the rounding.  Passing torch.bfloat16 here runs exactly that pair of operations -
    cast the logits, sigmoid in that dtype - in the middle of an otherwise higher-precision evaluation, so that
    the oracle sees the layer's decays and their gradients (zero where the decay rounds to one).

    Follows spear/nn/phalanx/swr.py:157-175 (the four projections), :96-103 (head h reads key/value head
    h // (heads / kv_heads)), :196-221 (A = sigmoid, X = sigmoid(B) * V), :311-327 (y * C + V, output
    projection).  `state` is the layer's state_dict (same parameter names as the reference's).
    """
    lin = lambda name, t: torch.nn.functional.linear(t, state[f"param.{name}.weight"].to(t.dtype),
                                                     None if f"param.{name}.bias" not in state
                                                     else state[f"param.{name}.bias"].to(t.dtype))
    Bsz, L, dim = u.shape
    H = state["param.proj_a.weight"].shape[0]
    D = state["param.proj_v.weight"].shape[0] // H
    KV = H if kv_heads is None else kv_heads
    idx = torch.arange(H) // (H // KV)
    heads = lambda t, n: t.transpose(1, 2).reshape(Bsz, n, D, L)
    a_logits = lin("proj_a", u)
    if decay_dtype is not None:
        A = torch.sigmoid(a_logits.to(decay_dtype)).to(u.dtype).transpose(1, 2)
    else:
        A = torch.sigmoid(a_logits).transpose(1, 2)
    Bg = heads(lin("proj_b", u), KV).index_select(1, idx)
    C = heads(lin("proj_c", u), KV).index_select(1, idx)
    V = heads(lin("proj_v", u), H)
    X = torch.sigmoid(Bg) * V
    y = btp_forward(A.contiguous(), X.contiguous(), k) * C + V
    y = y.reshape(Bsz, H * D, L).transpose(1, 2)
    return torch.nn.functional.linear(y, state["proj_out.weight"].to(u.dtype))
