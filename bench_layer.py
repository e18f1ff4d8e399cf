"""Timing of the gated (token-major) op and of the whole Phalanx layer, on one GPU or batch-sharded over several.

    python bench_layer.py [--batch 1024 --length 128 --dim 512] [--steps 50] [--what gated|layer|both]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench_layer.py --what layer --batch 64 --length 2048 --dim 2048 --decay-mix

Under torch.distributed.run `--batch` is the GLOBAL batch: each rank takes its slice (strong scaling, no
exchange on the forward/backward data path), times are the maximum over ranks and rank 0 prints.  With
`--allreduce-grads` each step also sums the parameter gradients over the ranks (one NCCL all-reduce of the
flattened gradients), which is what data-parallel training adds to the layer.

`gated`: one fused forward + one fused backward launch per step on resident inputs; reports time per
launch and achieved GB/s against the algorithmic bytes (forward 130 B, backward 228 B per head-token:
inputs read once, outputs written once).  `layer`: Phalanx forward+backward through autograd, with the
gating fused and, for comparison, operation by operation.  Synthetic N(0,1) inputs, CUDA events, rotating
input sets so that successive launches do not find their inputs in L2.  One JSON line per measurement.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

GATED_FWD_BYTES = 130  # per head-token: A 2 + B 32 + C 32 + V 32 read, out 32 written
GATED_BWD_BYTES = 228  # A 2 + B, C, V, dOut 128 read; dA 2 + dB, dC, dV 96 written


def _timed(fn, steps, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps * 1e3  # us


def bench_gated(B, L, H, steps, sets, kv=None):
    """kv: number of key/value heads (default H: every head its own); B_logits and C are [B, L, kv*16] then."""
    from spear_b200 import _lib
    from spear_b200.ops.btp import gated as G

    cols = H * 16
    kv = H if kv is None else kv
    data = []
    for _ in range(sets):
        al = torch.randn(B, L, H, device="cuda").bfloat16()
        bl, c = (torch.randn(B, L, kv * 16, device="cuda").bfloat16() for _ in range(2))
        v, do = (torch.randn(B, L, cols, device="cuda").bfloat16() for _ in range(2))
        data.append((al, bl, c, v, do, torch.empty_like(v)))
    i = [0]

    def fwd():
        al, bl, c, v, do, out = data[i[0] % sets]
        i[0] += 1
        G._launch_forward(al, bl, c, v, out, 2)

    def bwd():
        al, bl, c, v, do, out = data[i[0] % sets]
        i[0] += 1
        G._backward(al, bl, c, v, do, 2)

    ht = B * L * H
    tf, tb = _timed(fwd, steps), _timed(bwd, steps)
    _lib.device_status()
    # algorithmic bytes per head-token: shared B_logits / C are read once per key/value head, and the kernel
    # writes dB_logits / dC summed over the runs of heads it shares (see gated._shared_run)
    run = G._shared_run(H, kv)
    fwd_bytes = GATED_FWD_BYTES - 64 + 64 * kv / H
    bwd_bytes = GATED_BWD_BYTES - 64 + 64 * kv / H - 64 + 64 / run
    return {
        "what": "gated_btp", "B": B, "L": L, "H": H, "kv_heads": kv, "fwd_us": tf, "bwd_us": tb,
        "fwd_bytes_per_head_token": fwd_bytes, "bwd_bytes_per_head_token": bwd_bytes,
        "fwd_gbs": fwd_bytes * ht / tf / 1e3, "bwd_gbs": bwd_bytes * ht / tb / 1e3,
        "fwd_bwd_tokens_per_s": B * L / ((tf + tb) * 1e-6),
    }


def set_decay_mix(layer) -> None:
    """Input-independent decays: half the heads get log a ~ U(-1e-3, 0), the other half U(-4, -1)."""
    prm = layer.param
    H = prm.proj_a.bias.numel()
    g = torch.Generator().manual_seed(7)
    log_a = torch.cat([torch.rand(H // 2, generator=g) * -1e-3, -1.0 - 3.0 * torch.rand(H - H // 2, generator=g)])
    a = torch.exp(log_a.double()).clamp(max=1.0 - 1e-12)
    with torch.no_grad():
        prm.proj_a.weight.zero_()
        prm.proj_a.bias.copy_(torch.log(a / (1.0 - a)).to(prm.proj_a.bias.dtype))  # sigmoid(bias) = a


def bench_layer(B, L, dim, steps, *, decay_mix=False, allreduce_grads=False, rank=0, world=1):
    from spear_b200.nn.phalanx import Phalanx
    from spear_b200.sharding import batch_shard, max_over_ranks

    torch.manual_seed(0)  # every rank holds the same weights
    layer = Phalanx(dim=dim, length=L, dtype=torch.bfloat16).cuda()
    if decay_mix:
        set_decay_mix(layer)
    lo, hi = batch_shard(B, rank, world)
    torch.manual_seed(1 + rank)
    u = torch.randn(hi - lo, L, dim, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    do = torch.randn(hi - lo, L, dim, device="cuda", dtype=torch.bfloat16)
    params = list(layer.parameters())

    def step():
        layer.zero_grad(set_to_none=True)
        u.grad = None
        layer(u).backward(do)
        if allreduce_grads and world > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in params])
            torch.distributed.all_reduce(flat)

    out = {"what": "phalanx_layer_fwd_bwd", "global_batch": B, "L": L, "dim": dim, "n_gpus": world,
           "batch_per_gpu": hi - lo, "decay_mix": bool(decay_mix), "allreduce_grads": bool(allreduce_grads and world > 1)}
    for fused in (True, False):
        layer.fused_gating = fused
        if world > 1:
            torch.distributed.barrier()
        t = _timed(step, steps, warm=2)
        t = max_over_ranks([t], device="cuda")[0] if world > 1 else t
        out["fused_ms" if fused else "unfused_ms"] = t / 1e3
    out["tokens_per_s_fused"] = B * L / (out["fused_ms"] * 1e-3)
    out["speedup"] = out["unfused_ms"] / out["fused_ms"]
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1024)
    ap.add_argument("--length", type=int, default=128)
    ap.add_argument("--dim", type=int, default=512)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--sets", type=int, default=3)
    ap.add_argument("--what", default="both", choices=["gated", "layer", "both"])
    ap.add_argument("--kv-heads", type=int, default=None, help="gated: key/value heads shared by groups of heads")
    ap.add_argument("--decay-mix", action="store_true", help="layer: fixed decays, half the heads near 1, half fast")
    ap.add_argument("--allreduce-grads", action="store_true", help="layer, several ranks: sum parameter gradients each step")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    try:
        if args.what in ("gated", "both") and rank == 0:
            print(json.dumps(bench_gated(args.batch, args.length, args.dim // 16, args.steps, args.sets, args.kv_heads)), flush=True)
        if args.what in ("layer", "both"):
            res = bench_layer(args.batch, args.length, args.dim, max(3, args.steps // 10), decay_mix=args.decay_mix,
                              allreduce_grads=args.allreduce_grads, rank=rank, world=world)
            if rank == 0:
                print(json.dumps(res), flush=True)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
