"""``btp(coeff, x, k=2, wpb=None, output_dtype=None)`` on the sm_100a kernels.

Mirrors the reference wrapper (spear/ops/btp/interface.py:23-188): same
function signature and defaults, the same pair of mutating custom ops
``spear_btp::forward`` / ``spear_btp::backward`` (so ``torch.compile`` traces
it the same way), the same autograd contract (gradients ``dA`` float32 for
``coeff`` and ``dx`` in ``x.dtype``).

Differences, all deliberate:
* ``coeff.shape`` is validated (the reference never checks it, interface.py:136-139).
* no carry checkpoint is allocated or written: backward recomputes the carry.
* ``dA`` is not pre-zeroed: the kernel writes every element.
* ``coeff`` may also be float32, and with ``coeff_space="log"`` it is the natural
  log of the coefficient (float32) - a superset for decays that bf16 cannot hold.
* bfloat16 or float16 activations (as in the reference); there is no CPU path and no fallback.
"""

from __future__ import annotations

import torch
import torch.library

from ... import _btp as _native

__all__ = ["btp", "DH", "BLK", "SUPPORTED_WPB", "WPB_K1_DEFAULT", "WPB_K2_DEFAULT"]

# constants of spear/ops/btp/interface.py:23-27
DH = 16
BLK = 16
SUPPORTED_WPB = [4, 8, 16, 32]
WPB_K1_DEFAULT = 8
WPB_K2_DEFAULT = 32


def _forward_impl(coeff: torch.Tensor, x: torch.Tensor, y: torch.Tensor, checkpoint: torch.Tensor, k: int, wpb: int) -> None:
    _native.forward(coeff, x, y, checkpoint, k, wpb)


def _backward_impl(
    coeff: torch.Tensor, x: torch.Tensor, dy: torch.Tensor, checkpoint: torch.Tensor, dx: torch.Tensor, dA: torch.Tensor,
    k: int, wpb: int,
) -> None:
    _native.backward(coeff, x, dy, checkpoint, dx, dA, k, wpb)


def _forward_log_impl(coeff: torch.Tensor, x: torch.Tensor, y: torch.Tensor, checkpoint: torch.Tensor, k: int, wpb: int) -> None:
    _native.forward(coeff, x, y, checkpoint, k, wpb, log_coeff=True)


def _backward_log_impl(
    coeff: torch.Tensor, x: torch.Tensor, dy: torch.Tensor, checkpoint: torch.Tensor, dx: torch.Tensor, dA: torch.Tensor,
    k: int, wpb: int,
) -> None:
    _native.backward(coeff, x, dy, checkpoint, dx, dA, k, wpb, log_coeff=True)


def _fake_fwd(coeff, x, y, checkpoint, k, wpb) -> None:
    return None


def _fake_bwd(coeff, x, dy, checkpoint, dx, dA, k, wpb) -> None:
    return None


def _op_exists(ns: str, name: str) -> bool:
    try:
        getattr(getattr(torch.ops, ns), name)
        return True
    except (AttributeError, RuntimeError):
        return False


def _register(lib: torch.library.Library, ns: str, name: str, impl, fake, mutates) -> None:
    """Same registration as the reference's register_traceable_op (interface.py:36-52)."""
    if _op_exists(ns, name):  # e.g. the reference package was imported first in this process
        return
    schema = torch.library.infer_schema(impl, mutates_args=mutates)
    lib.define(name + schema)
    lib.impl(name, impl, "CUDA")
    lib._register_fake(name, fake)


_LIB = torch.library.Library("spear_btp", "FRAGMENT")
_register(_LIB, "spear_btp", "forward", _forward_impl, _fake_fwd, ["y", "checkpoint"])
_register(_LIB, "spear_btp", "backward", _backward_impl, _fake_bwd, ["dx", "dA"])
_register(_LIB, "spear_btp", "forward_log", _forward_log_impl, _fake_fwd, ["y", "checkpoint"])
_register(_LIB, "spear_btp", "backward_log", _backward_log_impl, _fake_bwd, ["dx", "dA"])


class _BTPFunction(torch.autograd.Function):
    """Autograd glue, same contract as interface.py:126-161."""

    @staticmethod
    def forward(ctx, coeff, x, k, output_dtype, wpb, log_space):
        B, H, dh_in, L = x.shape
        assert dh_in == DH, f"Channel dimension must be {DH}"
        assert L % BLK == 0, f"Length L must be multiple of {BLK}"
        assert wpb in SUPPORTED_WPB, f"WPB must be one of {SUPPORTED_WPB}"
        if tuple(coeff.shape) != (B, H, L):
            raise ValueError(f"coeff must have shape {(B, H, L)}, got {tuple(coeff.shape)}")

        y = torch.empty_like(x, dtype=output_dtype)
        checkpoint = torch.empty(0, device=x.device, dtype=torch.float32)  # not needed by these kernels
        if log_space:
            torch.ops.spear_btp.forward_log(coeff, x, y, checkpoint, int(k), int(wpb))
        else:
            torch.ops.spear_btp.forward(coeff, x, y, checkpoint, int(k), int(wpb))

        ctx.save_for_backward(coeff, x)
        ctx.k = int(k)
        ctx.wpb = int(wpb)
        ctx.log_space = bool(log_space)
        return y

    @staticmethod
    def backward(ctx, dy):
        coeff, x = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dA = torch.empty_like(coeff, dtype=torch.float32)
        checkpoint = torch.empty(0, device=x.device, dtype=torch.float32)
        if ctx.log_space:
            torch.ops.spear_btp.backward_log(coeff, x, dy, checkpoint, dx, dA, ctx.k, ctx.wpb)
        else:
            torch.ops.spear_btp.backward(coeff, x, dy, checkpoint, dx, dA, ctx.k, ctx.wpb)
        return dA, dx, None, None, None, None


def btp(
    coeff: torch.Tensor,
    x: torch.Tensor,
    k: int = 2,
    wpb: int | None = None,
    output_dtype: torch.dtype | None = None,
    *,
    coeff_space: str = "linear",
) -> torch.Tensor:
    """Block two-pass sliding-window recurrence (signature of interface.py:164-188).

    Args:
        coeff: [B, H, L] decay coefficients in (0, 1]; x's 16-bit type (as in the reference) or float32.
        x: [B, H, 16, L] bfloat16 or float16 driving term.
        k: 2 = local pass plus one-hop carry, 1 = local pass only.
        wpb: accepted for compatibility ({4, 8, 16, 32}); the kernels choose their own launch shape.
        output_dtype: dtype of the result, default float32 (as in the reference).
        coeff_space: "linear" (default) or "log" (coeff is log(a), float32).
    Returns:
        y: [B, H, 16, L] in ``output_dtype``.
    """
    if coeff_space not in ("linear", "log"):
        raise ValueError("coeff_space must be 'linear' or 'log'")
    if not (x.is_cuda and coeff.is_cuda):
        raise RuntimeError("btp needs CUDA tensors: this package has no CPU path and no fallback")
    out_dtype = output_dtype or torch.float32
    wpb_val = wpb if wpb is not None else (WPB_K2_DEFAULT if k == 2 else WPB_K1_DEFAULT)
    coeff = coeff.contiguous()
    x = x.contiguous()
    return _BTPFunction.apply(coeff, x, k, out_dtype, wpb_val, coeff_space == "log")
