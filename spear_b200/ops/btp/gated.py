"""Gated BTP in token-major layout: the Phalanx layer's glue fused around the op.

    out = btp(sigmoid(A_logits), sigmoid(B_logits) * V) * C + V

with every tensor laid out as the layer's projections produce it ([B, L, H] and [B, L, H*16]); replaces
spear/nn/phalanx/swr.py:216-219 and 320-323 plus the two transposing copies of
spear/ops/btp/interface.py:186-187.  CUDA only, bf16 only, no fallback.
"""

from __future__ import annotations

import ctypes

import torch

from ... import _btp as _native
from ... import _lib
from . import interface as _iface

__all__ = ["gated_btp", "gated_btp_wide", "gated_btp_supported"]


def gated_btp_supported(heads: int, kv_heads: int, length: int) -> bool:
    """The fused kernels take 4 heads per CTA.  Heads that share key/value heads (kv_heads < heads, KVRepeat of
    spear/nn/phalanx/swr.py:96-103) are supported for any divisor: the kernels read the shared B_logits and C
    columns in place."""
    return heads % 4 == 0 and heads % kv_heads == 0 and length % 16 == 0


def _rows(t: torch.Tensor, cols: int, what: str) -> int:
    """Row pitch (elements) of a [B, L, cols] tensor whose rows are dense and evenly spaced."""
    if t.dim() != 3 or t.shape[2] != cols:
        raise ValueError(f"{what} must be [B, L, {cols}], got {tuple(t.shape)}")
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA bfloat16 tensor (there is no CPU path)")
    B, L, _ = t.shape
    if t.stride(2) != 1 or (B > 1 and t.stride(0) != L * t.stride(1)):
        raise ValueError(f"{what}: rows must be dense and evenly spaced (strides {t.stride()})")
    return t.stride(1)


def _same_batch_and_length(a_logits: torch.Tensor, others) -> None:
    """Every [B, L, .] tensor of one call must share a_logits' B, L and device: the kernels build their
    descriptors over [B][L] from a_logits alone, so a shorter tensor would be read or written out of bounds."""
    if a_logits.dim() != 3:
        raise ValueError(f"a_logits must be [B, L, H], got {tuple(a_logits.shape)}")
    for t, name in others:
        if t.dim() != 3 or t.shape[:2] != a_logits.shape[:2]:
            raise ValueError(f"{name} must share a_logits' batch and length {tuple(a_logits.shape[:2])}, got {tuple(t.shape)}")
        if t.device != a_logits.device:
            raise ValueError(f"{name} is on {t.device}, a_logits on {a_logits.device}")


def _kv_heads(b_logits: torch.Tensor, c: torch.Tensor, H: int) -> int:
    """Number of key/value heads from the width of B_logits (C must agree); a divisor of H."""
    if b_logits.dim() != 3 or c.dim() != 3 or b_logits.shape[2] != c.shape[2]:
        raise ValueError(f"b_logits and c must be [B, L, kv_heads*16] of one width, got {tuple(b_logits.shape)}, {tuple(c.shape)}")
    kv, rest = divmod(b_logits.shape[2], 16)
    if rest or kv < 1 or H % kv:
        raise ValueError(f"b_logits has {b_logits.shape[2]} columns: not 16 per key/value head with kv_heads dividing {H} heads")
    return kv


def _shared_run(H: int, kv: int) -> int:
    """Over how many neighbouring heads the backward kernel itself sums dB_logits and dC: 4 when the group size
    H / kv is a multiple of 4 (the four heads of a CTA share one key/value head), 2 when it is 2, else 1."""
    group = H // kv
    return 4 if group % 4 == 0 else (2 if group == 2 else 1)


def _launch_forward(a_logits, b_logits, c, v, out, k: int) -> None:
    _same_batch_and_length(a_logits, ((b_logits, "b_logits"), (c, "c"), (v, "v"), (out, "out")))
    B, L, H = a_logits.shape
    cols = H * 16
    kv = _kv_heads(b_logits, c, H)
    ld_a = _rows(a_logits, H, "a_logits")
    ld_b, ld_c = _rows(b_logits, kv * 16, "b_logits"), _rows(c, kv * 16, "c")
    ld_v, ld_o = _rows(v, cols, "v"), _rows(out, cols, "out")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    with _native._OnDevice(v.device.index) as stream:
        rc = _lib.load().btp_sm100_gated_forward(p(a_logits), p(b_logits), p(c), p(v), p(out), B, L, H, kv, ld_a, ld_b,
                                                 ld_c, ld_v, ld_o, int(k), ctypes.c_void_p(stream))
    _lib.check(rc, "btp_sm100_gated_forward")


class _GatedBTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a_logits, b_logits, c, v, k):
        out = torch.empty(v.shape, device=v.device, dtype=v.dtype)
        torch.ops.spear_btp.gated_forward(a_logits, b_logits, c, v, out, int(k))
        ctx.save_for_backward(a_logits, b_logits, c, v)
        ctx.k = int(k)
        return out

    @staticmethod
    def backward(ctx, dout):
        a_logits, b_logits, c, v = ctx.saved_tensors
        return _backward(a_logits, b_logits, c, v, dout, ctx.k) + (None,)


def _launch_backward(a_logits, b_logits, c, v, dout, da, db, dc, dv, k: int) -> None:
    _same_batch_and_length(a_logits, ((b_logits, "b_logits"), (c, "c"), (v, "v"), (dout, "dout"), (da, "da_logits"),
                                      (db, "db_logits"), (dc, "dc"), (dv, "dv")))
    B, L, H = a_logits.shape
    cols = H * 16
    kv = _kv_heads(b_logits, c, H)
    ld = [_rows(a_logits, H, "a_logits"), _rows(b_logits, kv * 16, "b_logits"), _rows(c, kv * 16, "c"),
          _rows(v, cols, "v"), _rows(dout, cols, "dout")]
    # db and dc come out summed over the runs of heads that a CTA shares (see _shared_run): width H*16 / run
    gcols = cols // _shared_run(H, kv)
    ld += [_rows(da, H, "da_logits"), _rows(db, gcols, "db_logits"), _rows(dc, gcols, "dc"), _rows(dv, cols, "dv")]
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    with _native._OnDevice(v.device.index) as stream:
        rc = _lib.load().btp_sm100_gated_backward(p(a_logits), p(b_logits), p(c), p(v), p(dout), p(da), p(db), p(dc), p(dv),
                                                  B, L, H, kv, *ld, int(k), ctypes.c_void_p(stream))
    _lib.check(rc, "btp_sm100_gated_backward")


# ---- custom ops (mutating, with no-op fakes) so that torch.compile traces through them like through
#      spear_btp::forward / spear_btp::backward
def _op_gated_forward(a_logits: torch.Tensor, b_logits: torch.Tensor, c: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                      k: int) -> None:
    _launch_forward(a_logits, b_logits, c, v, out, k)


def _op_gated_backward(a_logits: torch.Tensor, b_logits: torch.Tensor, c: torch.Tensor, v: torch.Tensor, dout: torch.Tensor,
                       da: torch.Tensor, db: torch.Tensor, dc: torch.Tensor, dv: torch.Tensor, k: int) -> None:
    _launch_backward(a_logits, b_logits, c, v, dout, da, db, dc, dv, k)


def _op_gated_forward_wide(wide: torch.Tensor, out: torch.Tensor, heads: int, k: int) -> None:
    bl, c, v, al = _split_wide(wide, heads)
    _launch_forward(al, bl, c, v, out, k)


def _op_gated_backward_wide(wide: torch.Tensor, dout: torch.Tensor, dwide: torch.Tensor, heads: int, k: int) -> None:
    bl, c, v, al = _split_wide(wide, heads)
    db, dc, dv, da = _split_wide(dwide, heads)
    _launch_backward(al, bl, c, v, dout, da, db, dc, dv, k)


def _fake(*args) -> None:
    return None


_iface._register(_iface._LIB, "spear_btp", "gated_forward", _op_gated_forward, _fake, ["out"])
_iface._register(_iface._LIB, "spear_btp", "gated_backward", _op_gated_backward, _fake, ["da", "db", "dc", "dv"])
_iface._register(_iface._LIB, "spear_btp", "gated_forward_wide", _op_gated_forward_wide, _fake, ["out"])
_iface._register(_iface._LIB, "spear_btp", "gated_backward_wide", _op_gated_backward_wide, _fake, ["dwide"])


def _backward(a_logits, b_logits, c, v, dout, k):
    B, L, H = a_logits.shape
    cols = H * 16
    dout = dout if dout.stride(2) == 1 else dout.contiguous()
    kv = b_logits.shape[2] // 16
    run = _shared_run(H, kv)
    da = torch.empty(B, L, H, device=v.device, dtype=v.dtype)
    dv = torch.empty(B, L, cols, device=v.device, dtype=v.dtype)
    db, dc = (torch.empty(B, L, cols // run, device=v.device, dtype=v.dtype) for _ in range(2))
    torch.ops.spear_btp.gated_backward(a_logits, b_logits, c, v, dout, da, db, dc, dv, int(k))
    parts = H // kv // run  # partial sums per key/value head that the kernel left (1: nothing left to add)
    if parts > 1:
        db = db.view(B, L, kv, parts, 16).sum(dim=3).reshape(B, L, kv * 16)
        dc = dc.view(B, L, kv, parts, 16).sum(dim=3).reshape(B, L, kv * 16)
    return da, db, dc, dv


def _split_wide(wide: torch.Tensor, H: int):
    """Column slices (b_logits, c, v, a_logits) of a [B, L, 3*H*16 + H] projection output."""
    d = H * 16
    return wide[..., :d], wide[..., d:2 * d], wide[..., 2 * d:3 * d], wide[..., 3 * d:3 * d + H]


class _GatedBTPWide(torch.autograd.Function):
    """Same op on the output of ONE wide projection; the backward kernel writes the four gradients straight
    into the column slices of one gradient tensor, so nothing is concatenated or zero-filled."""

    @staticmethod
    def forward(ctx, wide, heads, k):
        B, L, _ = wide.shape
        out = torch.empty(B, L, heads * 16, device=wide.device, dtype=wide.dtype)
        torch.ops.spear_btp.gated_forward_wide(wide, out, int(heads), int(k))
        ctx.save_for_backward(wide)
        ctx.heads, ctx.k = int(heads), int(k)
        return out

    @staticmethod
    def backward(ctx, dout):
        (wide,) = ctx.saved_tensors
        dwide = torch.empty_like(wide)
        dout = dout if dout.stride(2) == 1 else dout.contiguous()
        torch.ops.spear_btp.gated_backward_wide(wide, dout, dwide, ctx.heads, ctx.k)
        return dwide, None, None


def gated_btp_wide(wide: torch.Tensor, heads: int, k: int = 2) -> torch.Tensor:
    """gated_btp on one projection output `wide` [B, L, 3*heads*16 + heads] whose columns are
    (b_logits | c | v | a_logits).  heads must be a multiple of 8 (16-byte aligned column slices)."""
    if wide.dim() != 3 or wide.shape[2] != 3 * heads * 16 + heads:
        raise ValueError(f"wide must be [B, L, {3 * heads * 16 + heads}], got {tuple(wide.shape)}")
    if heads % 8 != 0 or wide.shape[1] % 16 != 0:
        raise ValueError("gated_btp_wide needs heads % 8 == 0 and L % 16 == 0")
    if not wide.is_contiguous():
        wide = wide.contiguous()
    return _GatedBTPWide.apply(wide, heads, k)


def gated_btp(a_logits: torch.Tensor, b_logits: torch.Tensor, c: torch.Tensor, v: torch.Tensor, k: int = 2) -> torch.Tensor:
    """out[B, L, H*16] = btp(sigmoid(a_logits), sigmoid(b_logits) * v) * c + v, token-major throughout.

    a_logits: [B, L, H]; v: [B, L, H*16]; b_logits, c: [B, L, kv_heads*16] with kv_heads a divisor of H (kv_heads = H
    when every head has its own; otherwise head h uses key/value head h // (H / kv_heads) and the shared columns
    are read in place).  All CUDA bfloat16 with dense rows (they may be column slices of one wider projection
    output).  H must be a multiple of 4 and L a multiple of 16.
    """
    if a_logits.dim() != 3:
        raise ValueError("a_logits must be [B, L, H]")
    H = a_logits.shape[2]
    if not gated_btp_supported(H, _kv_heads(b_logits, c, H), a_logits.shape[1]):
        raise ValueError(f"gated_btp needs heads % 4 == 0 and L % 16 == 0 (got H={H}, L={a_logits.shape[1]})")
    return _GatedBTP.apply(a_logits, b_logits, c, v, k)
