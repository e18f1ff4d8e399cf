"""Batch sharding of the BTP path over the GPUs of one box.

Every (batch, head) sequence is independent, so N ranks each take a contiguous
slice of the batch and nothing is exchanged on the data path.  The only
collectives are the ones a checker or a benchmark needs afterwards: the maximum
of a timing over ranks and global error norms.  They run on whatever backend the
process group has (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist


def batch_shard(global_batch: int, rank: int, world: int) -> tuple[int, int]:
    """[start, stop) of `rank`'s slice; slices differ by at most one entry and cover the batch exactly."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if global_batch < 0:
        raise ValueError("global_batch must be >= 0")
    base, extra = divmod(global_batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def bind_to_gpu_numa_node(device_index: int) -> list[int]:
    """Restricts the calling process to the CPU cores next to GPU `device_index` (NVML's ideal CPU affinity).

    With several ranks on one box, pinned host buffers should live on the memory of the socket their GPU hangs
    off: pages are placed where the thread that first touches them runs, and a copy whose host pages sit on the
    other socket crosses the inter-socket link in addition to PCIe.  Call it before allocating and filling the
    pinned buffers.  Only the CPU affinity of this process is changed (a per-process setting); nothing is written
    to the GPU or the driver.  Returns the cores chosen, or [] when NVML or the affinity call is unavailable -
    the process then stays where it is.
    """
    import os

    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cores = [64 * w + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1]
        allowed = sorted(set(cores) & os.sched_getaffinity(0))
        if not allowed:
            return []
        os.sched_setaffinity(0, allowed)
        return allowed
    except Exception:
        return []


def _world(group=None) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def max_over_ranks(values, device=None, group=None) -> list[float]:
    """Element-wise maximum of a few floats over all ranks (timings are reported as the slowest rank)."""
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    if _world(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.tolist()


def sum_over_ranks(values, device=None, group=None) -> list[float]:
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    if _world(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t.tolist()


def global_rel_l2(got: torch.Tensor, want: torch.Tensor, group=None) -> float:
    """||got - want|| / ||want|| over the shards of all ranks (each rank passes its own shard)."""
    g = got.detach().double()
    w = want.detach().double()
    num, den = sum_over_ranks([(g - w).square().sum().item(), w.square().sum().item()], device=got.device, group=group)
    return math.sqrt(num) / math.sqrt(den) if den > 0 else math.sqrt(num)


# ---------------------------------------------------------------------------------------------------
# Sequence sharding: one long sequence split over the ranks along L.
#
# The op is a ONE-hop recurrence (a block only sees the block-local last token of the block before it),
# so a rank needs exactly one 16-token block from each neighbour: forward the left neighbour's last block
# of (coeff, x); backward additionally the right neighbour's first block of (coeff, dy).  The halo blocks
# are exchanged with point-to-point messages (NCCL over NVLink on GPUs), copied into local memory, and the
# ordinary kernels run on [halo | local | halo]; nothing is ever read from a peer's memory by a kernel.
# ---------------------------------------------------------------------------------------------------
HALO = 16


def _neighbour_exchange(send_left, send_right, group=None):
    """Sends `send_left` to rank-1 and `send_right` to rank+1 (either may be None); returns
    (from_left, from_right), None at the ends of the chain.  Shapes must agree across ranks."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ops, from_left, from_right = [], None, None
    peer = lambda r: dist.get_global_rank(group, r) if group is not None else r
    if rank > 0:
        if send_left is not None:
            ops.append(dist.P2POp(dist.isend, send_left.contiguous(), peer(rank - 1), group))
        if send_right is not None:  # what the left neighbour sends right has the shape of what we send right
            from_left = torch.empty_like(send_right)
            ops.append(dist.P2POp(dist.irecv, from_left, peer(rank - 1), group))
    if rank < world - 1:
        if send_right is not None:
            ops.append(dist.P2POp(dist.isend, send_right.contiguous(), peer(rank + 1), group))
        if send_left is not None:
            from_right = torch.empty_like(send_left)
            ops.append(dist.P2POp(dist.irecv, from_right, peer(rank + 1), group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return from_left, from_right


def _native_forward(coeff, x, k, out_dtype):
    from . import _btp

    y = torch.empty(x.shape, device=x.device, dtype=out_dtype)
    _btp.forward(coeff, x, y, None, k, 32)
    return y


def _native_backward(coeff, x, dy, k):
    from . import _btp

    dx = torch.empty_like(x)
    dA = torch.empty(coeff.shape, device=x.device, dtype=torch.float32)
    _btp.backward(coeff, x, dy, None, dx, dA, k, 32)
    return dA, dx


class _SequenceParallelBTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, coeff, x, k, out_dtype, group, impl):
        fwd = impl[0] if impl else _native_forward
        rank = dist.get_rank(group)
        # my last block goes right; I receive the left neighbour's last block
        left_c, _ = _neighbour_exchange(None, coeff[..., -HALO:], group)
        left_x, _ = _neighbour_exchange(None, x[..., -HALO:], group)
        if rank > 0:
            y = fwd(torch.cat([left_c, coeff], -1).contiguous(), torch.cat([left_x, x], -1).contiguous(), k, out_dtype)
            y = y[..., HALO:]
        else:
            y = fwd(coeff.contiguous(), x.contiguous(), k, out_dtype)
        ctx.save_for_backward(coeff, x, left_c if rank > 0 else None, left_x if rank > 0 else None)
        ctx.k, ctx.group, ctx.impl = k, group, impl
        return y.contiguous()

    @staticmethod
    def backward(ctx, dy):
        coeff, x, left_c, left_x = ctx.saved_tensors
        bwd = ctx.impl[1] if ctx.impl else _native_backward
        group = ctx.group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        # my first block of (coeff, dy) goes left; I receive the right neighbour's first block
        _, right_c = _neighbour_exchange(coeff[..., :HALO], None, group)
        _, right_dy = _neighbour_exchange(dy[..., :HALO], None, group)
        cs, xs, ds = [coeff], [x], [dy]
        lo = 0
        if rank > 0:  # left halo: real (coeff, x), no upstream gradient of its own
            cs.insert(0, left_c); xs.insert(0, left_x); ds.insert(0, torch.zeros_like(dy[..., :HALO]))
            lo = HALO
        if rank < world - 1:  # right halo: real (coeff, dy); its x does not reach the local gradients
            cs.append(right_c); xs.append(torch.zeros_like(x[..., :HALO])); ds.append(right_dy)
        dA, dx = bwd(torch.cat(cs, -1).contiguous(), torch.cat(xs, -1).contiguous(), torch.cat(ds, -1).contiguous(), ctx.k)
        L = coeff.shape[-1]
        return dA[..., lo:lo + L].contiguous(), dx[..., lo:lo + L].contiguous(), None, None, None, None


def btp_sequence_parallel(coeff, x, k: int = 2, output_dtype=None, group=None, _impl=None):
    """btp() on a sequence that is split along L over the ranks of `group` (rank r holds the r-th slice).

    coeff: [B, H, L_local], x: [B, H, 16, L_local] with L_local a multiple of 16 on every rank (slices may
    differ in length).  Returns this rank's slice of y; gradients flow to this rank's slices of coeff and x.
    Every rank must call it (forward and backward are collective).  `_impl` = (forward_fn, backward_fn)
    replaces the kernels in host-side tests.
    """
    if coeff.shape[-1] % HALO or coeff.shape[-1] < HALO:
        raise ValueError("every rank's slice must be a positive multiple of 16 tokens")
    if not (dist.is_available() and dist.is_initialized()):
        raise RuntimeError("btp_sequence_parallel needs an initialised process group")
    return _SequenceParallelBTP.apply(coeff, x, int(k), output_dtype or torch.float32, group, _impl)
