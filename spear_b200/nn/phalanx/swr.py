"""Phalanx sliding-window-recurrence layer on the sm_100a BTP kernels.

Same public surface as the reference layer (spear/nn/phalanx/swr.py:21-331):
``KVRepeat``, ``SigmoidA`` and ``Phalanx`` with the same constructor arguments,
the same parameter names (so a reference ``state_dict`` loads unchanged:
``param.proj_{a,b,c}.{weight,bias}``, ``param.proj_v.weight``, ``proj_out.weight``)
and the same forward math:

    A = sigmoid(proj_a u)            [B, H, L]       decay
    X = sigmoid(proj_b u) * proj_v u [B, H, 16, L]   driving term
    y = btp(A, X) * proj_c u + proj_v u,  out = proj_out(y)

Only ``method="default"`` (the CUDA kernels) exists here.  The reference's
``"pytorch"`` / ``"pytorch_linspace"`` methods are its CPU reference paths; this
package ships no CPU path, so asking for them raises.
"""

from __future__ import annotations

import torch
import torch.nn as nn

HEAD_DIM = 16


class KVRepeat(nn.Module):
    """Shares one key/value head among ``total_heads // kv_heads`` query heads (swr.py:21-126)."""

    def __init__(self, kv_heads: int, total_heads: int):
        super().__init__()
        if total_heads % kv_heads != 0:
            raise ValueError(f"total_heads ({total_heads}) must be divisible by kv_heads ({kv_heads})")
        self.kv_heads = kv_heads
        self.total_heads = total_heads
        self.kv_groups = total_heads // kv_heads
        self.enabled = kv_heads < total_heads
        if self.enabled:
            # head h reads kv head h // kv_groups; non-persistent like the reference (not in state_dict)
            self.register_buffer("kv_indices", torch.arange(total_heads) // self.kv_groups, persistent=False)

    def forward(self, tensor: torch.Tensor, pattern: str = "b h d l") -> torch.Tensor:
        return tensor.index_select(1, self.kv_indices) if self.enabled else tensor

    def reshape_for_kv(self, tensor: torch.Tensor, batch: int, head_dim: int, length: int) -> torch.Tensor:
        return tensor.view(batch, self.kv_heads, head_dim, length)

    def expand_and_reshape(self, tensor: torch.Tensor, batch: int, head_dim: int, length: int) -> torch.Tensor:
        return self.forward(self.reshape_for_kv(tensor, batch, head_dim, length))

    def expand_flat(self, tensor: torch.Tensor, head_dim: int) -> torch.Tensor:
        if not self.enabled:
            return tensor
        batch, _, length = tensor.shape
        return self.expand_and_reshape(tensor, batch, head_dim, length).reshape(batch, self.total_heads * head_dim, length)


class SigmoidA(nn.Module):
    """Sigmoid-gated parametrisation producing (A, X, C, V) (swr.py:129-221)."""

    def __init__(
        self,
        dim: int,
        heads: int,
        head_dim: int,
        dtype: torch.dtype = torch.bfloat16,
        mixed_precision: bool = True,
        kv_heads: int | None = None,
    ):
        super().__init__()
        self.dim = dim
        self.heads = heads
        self.head_dim = head_dim
        self.dtype = dtype
        self.compute_dtype = torch.bfloat16  # activations are always cast to bf16 (swr.py:146,170)
        self.kv_heads = heads if kv_heads is None else kv_heads
        if heads % self.kv_heads != 0:
            raise ValueError(f"heads ({heads}) must be divisible by kv_heads ({self.kv_heads})")
        self.kv_repeat = KVRepeat(self.kv_heads, heads)
        self.dim_bvc = 3 * heads * head_dim
        self.dim_a = heads
        self.proj_a = nn.Linear(dim, heads, bias=True, dtype=dtype)
        self.proj_b = nn.Linear(dim, self.kv_heads * head_dim, bias=True, dtype=dtype)
        self.proj_c = nn.Linear(dim, self.kv_heads * head_dim, bias=True, dtype=dtype)
        self.proj_v = nn.Linear(dim, heads * head_dim, bias=False, dtype=dtype)

    def _compute_base_projections(self, x: torch.Tensor):
        u = x.to(self.compute_dtype)
        return tuple(proj(u).transpose(1, 2) for proj in (self.proj_a, self.proj_b, self.proj_c, self.proj_v))

    def forward_fused_gates(self, x: torch.Tensor) -> torch.Tensor:
        """Packed [B, 3*H*D + H, L] tensor in the order (B_gate, V, C, A) (swr.py:177-194)."""
        A, Bk, Ck, V = self._compute_base_projections(x)
        return torch.cat([self.kv_repeat.expand_flat(Bk, self.head_dim), V, self.kv_repeat.expand_flat(Ck, self.head_dim), A], dim=1)

    def forward_axcv(self, x: torch.Tensor):
        """(A [B,H,L], X, C, V [B,H,D,L]) for the BTP op (swr.py:196-221)."""
        batch, length, _ = x.shape
        A_logits, B_logits, C_kv, V_flat = self._compute_base_projections(x)
        V = V_flat.view(batch, self.heads, self.head_dim, length)
        B_gate = self.kv_repeat.expand_and_reshape(B_logits, batch, self.head_dim, length)
        C = self.kv_repeat.expand_and_reshape(C_kv, batch, self.head_dim, length)
        A = torch.sigmoid(A_logits)
        X = torch.sigmoid(B_gate) * V
        return A, X, C, V


class _PackedProjections:
    """The four projection weights of SigmoidA (swr.py:157-164) as row slices of ONE [3*dim + heads, dim] matrix,
    and their biases as slices of one vector, so that the projections run as one GEMM without concatenating
    anything per call.

    The parameters stay what they are - the same nn.Parameter objects under the same names, so state_dict,
    load_state_dict and optimizers see no difference - but their storage is moved into the packed buffers:
    `p.data` becomes a view of the packed matrix.  In-place updates (optimizer steps, load_state_dict) then
    change the packed matrix directly.  Operations that give a parameter fresh storage (`.to()`, `.cuda()`,
    a dtype cast) break the link; `current()` notices (the view's address no longer lies in the buffer) and packs
    again.  Row order: proj_b | proj_c | proj_v | proj_a, the column order the gated kernel reads.
    """

    def __init__(self, prm: "SigmoidA"):
        self.weights = (prm.proj_b.weight, prm.proj_c.weight, prm.proj_v.weight, prm.proj_a.weight)
        self.biases = (prm.proj_b.bias, prm.proj_c.bias, None, prm.proj_a.bias)
        rows = [w.shape[0] for w in self.weights]
        self.offsets = [sum(rows[:i]) for i in range(5)]
        with torch.no_grad():
            self.weight = torch.cat([w.detach() for w in self.weights], dim=0)
            self.bias = torch.zeros(self.offsets[4], device=self.weight.device, dtype=self.weight.dtype)
            for i, (w, b) in enumerate(zip(self.weights, self.biases)):
                lo, hi = self.offsets[i], self.offsets[i + 1]
                w.data = self.weight[lo:hi]
                if b is not None:
                    self.bias[lo:hi] = b.detach()
                    b.data = self.bias[lo:hi]

    def intact(self, prm: "SigmoidA") -> bool:
        ws = (prm.proj_b.weight, prm.proj_c.weight, prm.proj_v.weight, prm.proj_a.weight)
        bs = (prm.proj_b.bias, prm.proj_c.bias, None, prm.proj_a.bias)
        if any(a is not b for a, b in zip(ws + bs, self.weights + self.biases)):
            return False
        esz, dim = self.weight.element_size(), self.weight.shape[1]
        for i, (w, b) in enumerate(zip(ws, bs)):
            if w.dtype != self.weight.dtype or w.device != self.weight.device:
                return False
            if w.data_ptr() != self.weight.data_ptr() + self.offsets[i] * dim * esz:
                return False
            if b is not None and b.data_ptr() != self.bias.data_ptr() + self.offsets[i] * esz:
                return False
        return True


class _WideProjection(torch.autograd.Function):
    """wide = u @ W^T + bias with W, bias the packed buffers; the gradient of W is formed by ONE GEMM and handed
    to the four parameters as its row slices."""

    @staticmethod
    def forward(ctx, u, weight, bias, offsets, w_b, w_c, w_v, w_a, b_b, b_c, b_a):
        ctx.save_for_backward(u, weight)
        ctx.offsets = offsets
        return nn.functional.linear(u, weight, bias)

    @staticmethod
    def backward(ctx, dwide):
        u, weight = ctx.saved_tensors
        o = ctx.offsets
        d2 = dwide.reshape(-1, dwide.shape[-1])
        du = (d2 @ weight).reshape(u.shape) if ctx.needs_input_grad[0] else None
        dw = d2.t() @ u.reshape(-1, u.shape[-1])
        db = d2.sum(dim=0)
        return (du, None, None, None, dw[o[0]:o[1]], dw[o[1]:o[2]], dw[o[2]:o[3]], dw[o[3]:o[4]],
                db[o[0]:o[1]], db[o[1]:o[2]], db[o[3]:o[4]])


class Phalanx(nn.Module):
    """Drop-in for spear.nn.phalanx.Phalanx (swr.py:224-331) running the sm_100a BTP kernels."""

    def __init__(
        self,
        dim: int,
        heads: int | None = None,
        length: int = 2048,
        method: str = "default",
        dtype: torch.dtype = torch.float32,
        k: int = 2,
        wpb: int = 32,
        output_dtype: torch.dtype | None = None,
        block_size: int = 16,
        kv_heads: int | None = None,
    ):
        super().__init__()
        if heads is None:
            if dim % HEAD_DIM != 0:
                raise ValueError(f"dim ({dim}) must be divisible by 16")
            heads = dim // HEAD_DIM
        else:
            if dim % heads != 0:
                raise ValueError(f"dim ({dim}) must be divisible by heads ({heads})")
            if dim // heads != HEAD_DIM:
                raise ValueError(f"head_dim must be 16, got {dim // heads}. Use heads=dim//16 or leave heads=None")
        if method not in ("default", "pytorch", "pytorch_linspace"):
            raise ValueError(f"method must be one of 'default', 'pytorch', 'pytorch_linspace', got {method}")
        if method != "default":
            raise NotImplementedError(
                f"method={method!r} is the reference's CPU/PyTorch path; this package only ships the CUDA kernels "
                "(method='default') and has no fallback"
            )
        self.dim = dim
        self.heads = heads
        self.head_dim = HEAD_DIM
        self.length = (length + 15) // 16 * 16
        self.method = method
        self.dtype = dtype
        self.compute_dtype = torch.bfloat16
        self.k = k
        self.wpb = wpb
        self.output_dtype = output_dtype if output_dtype is not None else dtype
        self.block_size = block_size
        self.kv_heads = kv_heads if kv_heads is not None else heads

        self.param = SigmoidA(dim, heads, self.head_dim, dtype=dtype, kv_heads=kv_heads)
        self.proj_out = nn.Linear(dim, dim, bias=False, dtype=dtype)

        from spear_b200.ops.btp import btp

        self.btp_module = btp
        self._forward_fn = self._forward_default
        # The gating around the op runs fused, in the projections' own token-major layout, whenever the kernel
        # supports the configuration; set to False for the reference's operation-by-operation data flow.
        self.fused_gating = True
        # With fused gating and heads % 8 == 0 the four projections (swr.py:157-175) run as ONE GEMM whose
        # output columns (b | c | v | a) the gated kernel reads in place; the parameters stay separate.
        self.fused_projection = True
        self._packed = None  # _PackedProjections, built on the first fused forward

    def _forward_fused(self, x: torch.Tensor) -> torch.Tensor:
        from spear_b200.ops.btp.gated import gated_btp, gated_btp_wide

        u = x.to(self.compute_dtype)
        prm = self.param
        if self.kv_heads < self.heads:
            # Heads share key/value heads (KVRepeat, swr.py:96-103: head h reads key/value head h // group): the
            # gated kernels read the narrow B_logits and C in place, nothing is repeated.
            y = gated_btp(prm.proj_a(u), prm.proj_b(u), prm.proj_c(u), prm.proj_v(u), self.k)
        elif self.fused_projection and self.heads % 8 == 0:
            if torch.compiler.is_compiling():
                # under torch.compile the concatenation is traced (and fused) like any other op
                weight = torch.cat([prm.proj_b.weight, prm.proj_c.weight, prm.proj_v.weight, prm.proj_a.weight], dim=0)
                bias = torch.cat([prm.proj_b.bias, prm.proj_c.bias, torch.zeros_like(prm.proj_b.bias), prm.proj_a.bias])
                wide = nn.functional.linear(u, weight, bias)
            else:
                pk = self._packed
                if pk is None or not pk.intact(prm):
                    pk = self._packed = _PackedProjections(prm)
                wide = _WideProjection.apply(u, pk.weight, pk.bias, pk.offsets, prm.proj_b.weight, prm.proj_c.weight,
                                             prm.proj_v.weight, prm.proj_a.weight, prm.proj_b.bias, prm.proj_c.bias,
                                             prm.proj_a.bias)
            y = gated_btp_wide(wide, self.heads, self.k)
        else:
            y = gated_btp(prm.proj_a(u), prm.proj_b(u), prm.proj_c(u), prm.proj_v(u), self.k)
        return self.proj_out(y)

    def _forward_default(self, x: torch.Tensor) -> torch.Tensor:
        from spear_b200.ops.btp.gated import gated_btp_supported

        if (self.fused_gating and x.is_cuda and self.output_dtype == torch.bfloat16 and self.dtype == torch.bfloat16
                and gated_btp_supported(self.heads, self.kv_heads, x.shape[1])):
            return self._forward_fused(x)
        A, X, C, V = self.param.forward_axcv(x)
        y = self.btp_module(A, X, self.k, self.wpb, self.output_dtype)
        y = y * C + V
        batch, heads, head_dim, length = y.shape
        y = y.permute(0, 3, 1, 2).reshape(batch, length, heads * head_dim)
        return self.proj_out(y)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._forward_fn(x)
