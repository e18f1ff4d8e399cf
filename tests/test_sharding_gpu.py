"""Sequence sharding over two GPUs: NCCL halo exchange + the real kernels, against the full-sequence
oracle.  Needs two GPUs on the box (skipped otherwise)."""

from __future__ import annotations

import json
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import btp_oracle as O
    from spear_b200.sharding import btp_sequence_parallel, global_rel_l2

    g = torch.Generator().manual_seed(19)
    B, H, L = 2, 4, 4096
    a = torch.sigmoid(torch.randn(B, H, L, generator=g)).bfloat16()
    x = torch.randn(B, H, 16, L, generator=g).bfloat16()
    dy = torch.randn(B, H, 16, L, generator=g).bfloat16()
    cuts = [0, 1536, 4096]
    lo, hi = cuts[rank], cuts[rank + 1]
    al = a[..., lo:hi].cuda().contiguous().requires_grad_(True)
    xl = x[..., lo:hi].cuda().contiguous().requires_grad_(True)
    y = btp_sequence_parallel(al, xl, 2, torch.bfloat16)
    y.backward(dy[..., lo:hi].cuda().contiguous())
    torch.cuda.synchronize()
    y_w = O.btp_forward(a.float(), x.float())
    dA_w, dx_w = O.btp_backward(a.float(), x.float(), dy.float())
    res = {
        "y": global_rel_l2(y.detach().float(), y_w[..., lo:hi].cuda()),
        "dx": global_rel_l2(xl.grad.float(), dx_w[..., lo:hi].cuda()),
        "dA": global_rel_l2(al.grad.float(), dA_w[..., lo:hi].cuda()),
    }
    if rank == 0:
        json.dump(res, open(out, "w"))
    dist.destroy_process_group()


def test_sequence_sharding_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "res.json")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = json.load(open(out))
    assert all(v <= 1e-2 for v in res.values()), res
