"""Drop-in for the reference's compiled extension module ``spear._btp``.

Same two functions, same positional arguments, same in-place contract
(csrc/btp/_bindings.cu:76-229, 240-243):

    forward (coeff, x, y, checkpoint, k, wpb) -> None
    backward(coeff, x, dy, checkpoint, dx, dA, k, wpb) -> None

so that ``sys.modules["spear._btp"] = spear_b200._btp`` makes the unmodified
reference package run on these kernels.  The checks mirror the reference's
TORCH_CHECKs (_bindings.cu:19-60) and add the ones it lacks (coeff shape,
contiguity).  ``wpb`` is validated and otherwise ignored: the sm_100a kernels
pick their own launch shape.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib

DH = 16
BLK = 16
SUPPORTED_WPB = (4, 8, 16, 32)

_TAG = {torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32, torch.float16: _lib.DTYPE_F16}
_ACT = (torch.bfloat16, torch.float16)  # activation types of the kernels (the reference's, _bindings.cu:29-31)
_STREAM_TAG = {torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32}  # storage types of the streaming kernels


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


try:  # the raw-stream lookup that compiled launchers use; a few hundred ns instead of a Stream object
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:  # pragma: no cover
    def _raw_stream(index: int) -> int:
        return torch.cuda.current_stream(index).cuda_stream


class _OnDevice:
    """Makes `index` the current CUDA device for the call, only if it is not already."""

    __slots__ = ("index", "prev")

    def __init__(self, index: int):
        self.index = index
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.index:
            self.prev = cur
            torch.cuda.set_device(self.index)
        return _raw_stream(self.index)

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _ptr(t: torch.Tensor | None):
    """Address of a tensor's data as ctypes takes it for a void* argument (None = NULL); no wrapper object."""
    return None if t is None or t.numel() == 0 else t.data_ptr()


_current_device = torch.cuda.current_device


def _check_common(coeff: torch.Tensor, x: torch.Tensor, k: int, wpb: int) -> tuple[int, int, int]:
    # plain `if`s: the messages are only formatted when a check fails (this runs on every call)
    if not (x.is_cuda and coeff.is_cuda):
        raise RuntimeError("BTP tensors must be CUDA tensors (there is no CPU path)")
    if x.dim() != 4 or x.shape[2] != DH:
        raise RuntimeError(f"x must be [B, H, {DH}, L], got {tuple(x.shape)}")
    B, H, _, L = x.shape
    if coeff.shape != (B, H, L):
        raise RuntimeError(f"coeff must be [B, H, L] = {(B, H, L)}, got {tuple(coeff.shape)}")
    if L % BLK != 0:
        raise RuntimeError(f"Length L must be multiple of {BLK}")
    if k != 1 and k != 2:
        raise RuntimeError("k must be 1 or 2")
    if wpb not in SUPPORTED_WPB:
        raise RuntimeError(f"WPB must be one of {list(SUPPORTED_WPB)}")
    if x.dtype not in _ACT:
        raise RuntimeError(f"x must be bfloat16 or float16 (got {x.dtype})")
    if coeff.dtype != x.dtype and coeff.dtype != torch.float32:
        raise RuntimeError(f"coeff must have x's dtype ({x.dtype}) or be float32 (got {coeff.dtype})")
    if not (x.is_contiguous() and coeff.is_contiguous()):
        raise RuntimeError("coeff and x must be contiguous")
    if coeff.device != x.device:
        raise RuntimeError("coeff and x must be on the same device")
    return B, H, L


def _coeff_tag(coeff: torch.Tensor, x: torch.Tensor, log_coeff: bool) -> int:
    """Coefficient tag of the C ABI; a float coefficient carries the flag that says the activations are float16."""
    tag = _lib.DTYPE_F32_LOG if log_coeff else _TAG[coeff.dtype]
    if x.dtype == torch.float16 and coeff.dtype == torch.float32:
        tag |= _lib.ACT_F16
    return tag


def forward(coeff, x, y, checkpoint, k: int, wpb: int, *, log_coeff: bool = False) -> None:
    """y <- btp(coeff, x); optionally fills the reference's carry checkpoint."""
    B, H, L = _check_common(coeff, x, k, wpb)
    if y.shape != x.shape or not y.is_contiguous() or y.device != x.device:
        raise RuntimeError("y must match x and be contiguous")
    if y.dtype != torch.float32 and y.dtype != x.dtype:
        raise RuntimeError(f"y must be float32 or have x's dtype (got {y.dtype})")
    ytag = _TAG[y.dtype]
    if checkpoint is not None and checkpoint.numel():
        if checkpoint.dtype != torch.float32 or not checkpoint.is_contiguous():
            raise RuntimeError("checkpoint must be contiguous float32")
        if checkpoint.shape != (B, H, L // BLK, DH):
            raise RuntimeError("checkpoint must be [B, H, L/16, 16]")
    if log_coeff and coeff.dtype != torch.float32:
        raise RuntimeError("log-space coefficients must be float32")
    ctag = _coeff_tag(coeff, x, log_coeff)
    if x.numel() == 0:  # nothing to compute (empty batch, no heads or no tokens)
        return
    index = x.device.index
    fn = (_lib._lib or _lib.load()).btp_sm100_forward
    if index == _current_device():  # the usual case, without the context manager's overhead
        rc = fn(coeff.data_ptr(), x.data_ptr(), y.data_ptr(), _ptr(checkpoint), B, H, L, int(k), ctag, ytag, _raw_stream(index))
    else:
        with _OnDevice(index) as stream:
            rc = fn(coeff.data_ptr(), x.data_ptr(), y.data_ptr(), _ptr(checkpoint), B, H, L, int(k), ctag, ytag, stream)
    if rc:
        _lib.check(rc, "btp_sm100_forward")


def backward(coeff, x, dy, checkpoint, dx, dA, k: int, wpb: int, *, log_coeff: bool = False) -> None:
    """dx, dA <- gradients for upstream dy.  `checkpoint` is accepted and ignored."""
    B, H, L = _check_common(coeff, x, k, wpb)
    if dy.shape != x.shape or not dy.is_contiguous() or dy.device != x.device:
        raise RuntimeError("dy must match x and be contiguous")
    if dy.dtype != torch.float32 and dy.dtype != x.dtype:
        raise RuntimeError(f"dy must be float32 or have x's dtype (got {dy.dtype})")
    dytag = _TAG[dy.dtype]
    if dx.shape != x.shape or dx.dtype != x.dtype or not dx.is_contiguous():
        raise RuntimeError("dx must match x (shape, dtype)")
    if dA.shape != (B, H, L) or dA.dtype != torch.float32 or not dA.is_contiguous():
        raise RuntimeError("dA must be float32 [B, H, L]")
    if log_coeff and coeff.dtype != torch.float32:
        raise RuntimeError("log-space coefficients must be float32")
    ctag = _coeff_tag(coeff, x, log_coeff)
    if x.numel() == 0:
        return
    index = x.device.index
    fn = (_lib._lib or _lib.load()).btp_sm100_backward
    if index == _current_device():
        rc = fn(coeff.data_ptr(), x.data_ptr(), dy.data_ptr(), None, dx.data_ptr(), dA.data_ptr(), B, H, L, int(k), ctag, dytag,
                _raw_stream(index))
    else:
        with _OnDevice(index) as stream:
            rc = fn(coeff.data_ptr(), x.data_ptr(), dy.data_ptr(), None, dx.data_ptr(), dA.data_ptr(), B, H, L, int(k), ctag,
                    dytag, stream)
    if rc:
        _lib.check(rc, "btp_sm100_backward")


def decode_step(a_t, x_t, c_t, v_t, y_t, h_loc, r_pref, c_prev_loc, h_loc_out, r_pref_out, c_prev_loc_out, *,
                block_complete: bool, gate_is_log: bool, r_is_log: bool, _checked: bool = False) -> None:
    """One streaming step in one launch (btp_sm100_decode_step).  No counterpart in ``spear._btp``: the reference
    does this with tensor ops (spear/nn/phalanx/inference.py:177-266).  All tensors contiguous, [.., 16] ones of one
    dtype (bfloat16 or float32), a_t / r_pref / r_pref_out of one dtype (bfloat16 or float32)."""
    if not _checked:  # step_jagged builds every tensor itself and skips this
        big = (x_t, c_t, v_t, y_t, h_loc, c_prev_loc, h_loc_out) + (() if c_prev_loc_out is None else (c_prev_loc_out,))
        small = (a_t, r_pref_out) + (() if r_pref is None else (r_pref,))
        _require(all(t.is_cuda for t in big + small), "decode_step needs CUDA tensors (there is no CPU path)")
        _require(x_t.dim() >= 1 and x_t.shape[-1] == DH, f"x_t must be [..., {DH}]")
        _require(all(t.shape == x_t.shape and t.dtype == x_t.dtype and t.is_contiguous() for t in big),
                 "x_t, c_t, v_t, y_t and the [.,16] states must share shape and dtype and be contiguous")
        _require(all(t.shape == x_t.shape[:-1] and t.dtype == a_t.dtype and t.is_contiguous() for t in small),
                 "a_t and the r_pref states must be [...] of one dtype and contiguous")
        _require(x_t.dtype in _STREAM_TAG and a_t.dtype in _STREAM_TAG, "decode_step takes bfloat16 or float32 tensors")
        _require(not block_complete or c_prev_loc_out is not None, "the step that completes a block writes c_prev_loc_out")
    n_heads = a_t.numel()
    if n_heads == 0:
        return
    with _OnDevice(x_t.device.index) as stream:
        rc = _lib.load().btp_sm100_decode_step(
            _ptr(a_t), _ptr(x_t), _ptr(c_t), _ptr(v_t), _ptr(y_t), _ptr(h_loc), _ptr(r_pref), _ptr(c_prev_loc),
            _ptr(h_loc_out), _ptr(r_pref_out), _ptr(c_prev_loc_out), n_heads, int(block_complete), int(gate_is_log),
            int(r_is_log), _STREAM_TAG[x_t.dtype], _STREAM_TAG[a_t.dtype], ctypes.c_void_p(stream),
        )
    _lib.check(rc, "btp_sm100_decode_step")


def prefill_state(a, x, h_loc, r_pref, c_prev_loc, *, gate_is_log: bool) -> None:
    """Hand-off state after a prompt (btp_sm100_prefill_state; spear/nn/phalanx/inference.py:333-358).
    a [B,H,L], x [B,H,16,L] contiguous; outputs [B,H,16], [B,H], [B,H,16]."""
    _require(all(t.is_cuda for t in (a, x, h_loc, r_pref, c_prev_loc)), "prefill_state needs CUDA tensors (there is no CPU path)")
    _require(x.dim() == 4 and x.shape[2] == DH, f"x must be [B, H, {DH}, L]")
    B, H, _, L = x.shape
    _require(tuple(a.shape) == (B, H, L) and a.is_contiguous() and x.is_contiguous(), "a must be contiguous [B, H, L], x contiguous")
    _require(L >= 1, "the prompt must hold at least one token")
    for t in (h_loc, c_prev_loc):
        _require(tuple(t.shape) == (B, H, DH) and t.dtype == x.dtype and t.is_contiguous(), "h_loc, c_prev_loc must be [B, H, 16] of x's dtype")
    _require(tuple(r_pref.shape) == (B, H) and r_pref.dtype == a.dtype and r_pref.is_contiguous(), "r_pref must be [B, H] of a's dtype")
    _require(x.dtype in _STREAM_TAG and a.dtype in _STREAM_TAG, "prefill_state takes bfloat16 or float32 tensors")
    if B * H == 0:
        return
    with _OnDevice(x.device.index) as stream:
        rc = _lib.load().btp_sm100_prefill_state(
            _ptr(a), _ptr(x), _ptr(h_loc), _ptr(r_pref), _ptr(c_prev_loc), B * H, L, int(gate_is_log),
            _STREAM_TAG[x.dtype], _STREAM_TAG[a.dtype], ctypes.c_void_p(stream),
        )
    _lib.check(rc, "btp_sm100_prefill_state")
