"""Batch sharding and the checker's collectives with two gloo ranks on CPU."""

from __future__ import annotations

import json
import os
import socket
import subprocess
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shards_cover_the_batch_exactly():
    from spear_b200.sharding import batch_shard

    for B in (0, 1, 7, 64, 1024, 1025):
        for world in (1, 2, 3, 4, 8):
            spans = [batch_shard(B, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        batch_shard(8, 2, 2)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import btp_oracle as O
    from spear_b200.sharding import batch_shard, global_rel_l2, max_over_ranks, sum_over_ranks

    g = torch.Generator().manual_seed(5)
    B, H, L = 6, 2, 32
    a = torch.sigmoid(torch.randn(B, H, L, generator=g))
    x = torch.randn(B, H, 16, L, generator=g)
    lo, hi = batch_shard(B, rank, world)
    y_shard = O.btp_forward(a[lo:hi], x[lo:hi])          # every rank computes its own slice only
    y_full = O.btp_forward(a, x)
    noisy = y_shard + 1e-3 * (rank + 1)
    res = {
        "max": max_over_ranks([1.0 + rank, 5.0 - rank]),
        "sum": sum_over_ranks([hi - lo]),
        "rel_exact": global_rel_l2(y_shard, y_full[lo:hi]),
        "rel_noisy": global_rel_l2(noisy, y_full[lo:hi]),
    }
    # reference value of the noisy norm, computed centrally
    full_noisy = torch.cat([y_full[slice(*batch_shard(B, r, world))] + 1e-3 * (r + 1) for r in range(world)])
    res["rel_noisy_central"] = O.rel_l2(full_noisy, y_full)
    if rank == 0:
        json.dump(res, open(out, "w"))
    dist.destroy_process_group()


def test_two_gloo_ranks(tmp_path):
    out = str(tmp_path / "res.json")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = json.load(open(out))
    assert res["max"] == [2.0, 5.0]
    assert res["sum"] == [6.0]
    assert res["rel_exact"] == 0.0
    assert abs(res["rel_noisy"] - res["rel_noisy_central"]) < 1e-12


def test_reference_arm_prints_on_rank_zero_only():
    """bench.py --impl reference under two ranks: rank 0 prints the one JSON line, rank 1 exits 0 silently."""
    env = dict(os.environ, WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), OMP_NUM_THREADS="2")
    outs = []
    for rank in (0, 1):
        e = dict(env, RANK=str(rank), LOCAL_RANK=str(rank))
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                            "--steps", "1", "--warmup", "0", "--batch", "8"], env=e, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr
        outs.append(r.stdout.strip())
    assert outs[1] == ""
    line = json.loads(outs[0])
    staged = os.path.exists(os.path.join(ROOT, "oracle", "_ref", "spear", "ops", "btp", "reference.py"))
    # the reference's own code where it has been staged, the oracle port only where it has not
    assert line["impl"] == "reference" and line["n_gpus"] == 2
    assert line["cpu_baseline"]["kind"] == ("reference" if staged else "port")
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0


def _seq_worker(rank, world, port, out):
    """Two gloo ranks, each with a slice of L; the oracle stands in for the kernels (host-side logic only)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import btp_oracle as O
    from spear_b200.sharding import btp_sequence_parallel

    g = torch.Generator().manual_seed(9)
    B, H, L = 2, 3, 112
    a = torch.sigmoid(torch.randn(B, H, L, generator=g, dtype=torch.float64))
    x = torch.randn(B, H, 16, L, generator=g, dtype=torch.float64)
    dy = torch.randn(B, H, 16, L, generator=g, dtype=torch.float64)
    cuts = [0, 48, 112] if world == 2 else [0, 32, 64, 112]   # uneven slices
    lo, hi = cuts[rank], cuts[rank + 1]
    impl = (lambda c, xx, k, dt: O.btp_forward(c, xx, k, "product"),
            lambda c, xx, d, k: O.btp_backward(c, xx, d, k, "product"))
    al = a[..., lo:hi].clone().requires_grad_(True)
    xl = x[..., lo:hi].clone().requires_grad_(True)
    y = btp_sequence_parallel(al, xl, 2, torch.float64, None, impl)
    y.backward(dy[..., lo:hi])
    y_full = O.btp_forward(a, x, 2, "product")
    dA_full, dx_full = O.btp_backward(a, x, dy, 2, "product")
    res = {
        "y": (y.detach() - y_full[..., lo:hi]).abs().max().item(),
        "dx": (xl.grad - dx_full[..., lo:hi]).abs().max().item(),
        "dA": (al.grad - dA_full[..., lo:hi]).abs().max().item(),
    }
    json.dump(res, open(f"{out}.{rank}", "w"))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_sharding_with_halo_exchange(tmp_path, world):
    out = str(tmp_path / "seq")
    mp.spawn(_seq_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for rank in range(world):
        res = json.load(open(f"{out}.{rank}"))
        assert max(res.values()) < 1e-12, (rank, res)


def test_bind_to_gpu_numa_node_uses_the_affinity_nvml_reports(monkeypatch):
    """With a stand-in for NVML: the process ends up on the reported cores that it is allowed to use, and a
    missing NVML leaves it where it is."""
    import types

    from spear_b200.sharding import bind_to_gpu_numa_node

    before = os.sched_getaffinity(0)
    first = min(before)
    fake = types.ModuleType("pynvml")
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByIndex = lambda i: i
    fake.nvmlDeviceGetCpuAffinity = lambda h, words: [(1 << (first % 64)) if w == first // 64 else 0 for w in range(words)]
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    try:
        assert bind_to_gpu_numa_node(0) == [first]
        assert os.sched_getaffinity(0) == {first}
    finally:
        os.sched_setaffinity(0, before)
    fake.nvmlDeviceGetCpuAffinity = lambda h, words: [0] * words  # no usable core reported: nothing changes
    assert bind_to_gpu_numa_node(0) == [] and os.sched_getaffinity(0) == before
    monkeypatch.setitem(sys.modules, "pynvml", None)  # import fails
    assert bind_to_gpu_numa_node(0) == [] and os.sched_getaffinity(0) == before
