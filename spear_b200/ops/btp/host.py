"""BTP forward + backward for data that lives in HOST memory.

A training step whose activations are offloaded to (pinned) host memory pays for two PCIe transfers around
the kernels.  Run back to back (copy in, compute, copy out) the two directions of the link are never busy at
the same time.  `btp_fwd_bwd_host` cuts the batch into slices and runs three streams - host-to-device,
compute, device-to-host - so that the upload of slice i+1, the kernels of slice i and the download of slice
i-1 overlap; the step then costs about the larger of the two transfer times instead of their sum.
The kernels are the same C-ABI entry points that `btp()` calls; there is no CPU computation anywhere.
"""

from __future__ import annotations

import torch

from ... import _btp as _native

__all__ = ["btp_fwd_bwd_host"]


class _Ring:
    """Device buffers for `depth` slices in flight."""

    def __init__(self, depth, nb, H, L, x_dtype, coeff_dtype, dy_dtype, y_dtype, device):
        mk = lambda shape, dt: [torch.empty(shape, device=device, dtype=dt) for _ in range(depth)]
        self.a = mk((nb, H, L), coeff_dtype)
        self.x = mk((nb, H, 16, L), x_dtype)
        self.dy = mk((nb, H, 16, L), dy_dtype)
        self.y = mk((nb, H, 16, L), y_dtype)
        self.dx = mk((nb, H, 16, L), x_dtype)
        self.dA = mk((nb, H, L), torch.float32)
        self.free = [torch.cuda.Event() for _ in range(depth)]  # slice buffers fully downloaded


_rings: dict = {}


@torch.no_grad()
def btp_fwd_bwd_host(coeff, x, dy, y, dx, dA, *, k: int = 2, slices: int = 8, depth: int = 3, device=None):
    """y = btp(coeff, x); (dx, dA) = its gradients for upstream dy - all six tensors in pinned host memory.

    coeff [B,H,L] (x's 16-bit type or fp32), x, dy [B,H,16,L] (x bf16 or fp16; dy x's type or fp32) are read;
    y (x's type or fp32), dx (x's type), dA (fp32) are written.  The batch is processed in `slices` pieces with `depth` of them in
    flight.  Returns after enqueueing; synchronise the device (or the current stream) before reading the outputs.
    """
    if any(t.is_cuda for t in (coeff, x, dy, y, dx, dA)):
        raise ValueError("btp_fwd_bwd_host takes host tensors; use btp() for device tensors")
    if not all(t.is_pinned() for t in (coeff, x, dy, y, dx, dA)):
        raise ValueError("the host tensors must be pinned (page-locked) for the copies to overlap")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H, D, L = x.shape
    slices = max(1, min(slices, B))
    nb = (B + slices - 1) // slices
    key = (device.index, depth, nb, H, L, x.dtype, coeff.dtype, dy.dtype, y.dtype)
    ring = _rings.get(key)
    if ring is None:
        _rings.clear()  # one shape at a time: do not hoard device memory
        ring = _rings[key] = _Ring(depth, nb, H, L, x.dtype, coeff.dtype, dy.dtype, y.dtype, device)
        ring.streams = (torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device))
    s_in, s_run, s_out = ring.streams
    caller = torch.cuda.current_stream(device)
    for st in ring.streams:
        st.wait_stream(caller)
    for i in range(slices):
        lo, hi = i * nb, min(B, (i + 1) * nb)
        if lo >= hi:
            break
        n, r = hi - lo, i % depth
        up_x, up_dy, fwd_done, done = (torch.cuda.Event() for _ in range(4))
        with torch.cuda.stream(s_in):
            s_in.wait_event(ring.free[r])  # the previous occupant of these buffers has been downloaded
            ring.a[r][:n].copy_(coeff[lo:hi], non_blocking=True)
            ring.x[r][:n].copy_(x[lo:hi], non_blocking=True)
            up_x.record(s_in)              # forward can start while dy is still on its way
            ring.dy[r][:n].copy_(dy[lo:hi], non_blocking=True)
            up_dy.record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(up_x)
            _native.forward(ring.a[r][:n], ring.x[r][:n], ring.y[r][:n], None, k, 32)
            fwd_done.record(s_run)
            s_run.wait_event(up_dy)
            _native.backward(ring.a[r][:n], ring.x[r][:n], ring.dy[r][:n], None, ring.dx[r][:n], ring.dA[r][:n], k, 32)
            done.record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(fwd_done)     # y leaves while backward runs
            y[lo:hi].copy_(ring.y[r][:n], non_blocking=True)
            s_out.wait_event(done)
            dx[lo:hi].copy_(ring.dx[r][:n], non_blocking=True)
            dA[lo:hi].copy_(ring.dA[r][:n], non_blocking=True)
            ring.free[r].record(s_out)
    for st in ring.streams:
        caller.wait_stream(st)
