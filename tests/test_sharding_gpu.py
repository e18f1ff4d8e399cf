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


def test_one_process_driving_two_devices():
    """A single process alternating between cuda:0 and cuda:1 (per-device launch state, descriptors and the
    built-in scratch of the no-allocation entry are kept per device): every call runs on the device its tensors
    live on, whichever device is current, and both devices give the same results for the same inputs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ctypes

    import btp_oracle as O
    from spear_b200 import _lib
    from spear_b200.nn.phalanx import Phalanx
    from spear_b200.ops.btp import btp

    g = torch.Generator().manual_seed(23)
    B, H, L = 3, 8, 400
    a = torch.sigmoid(torch.randn(B, H, L, generator=g)).bfloat16()
    x = torch.randn(B, H, 16, L, generator=g).bfloat16()
    dy = torch.randn(B, H, 16, L, generator=g).bfloat16()
    y_w = O.btp_forward(a.float(), x.float())
    dA_w, dx_w = O.btp_backward(a.float(), x.float(), dy.float())
    outs = {}
    for current, target in ((0, 1), (1, 0), (1, 1), (0, 0)):
        torch.cuda.set_device(current)
        dev = torch.device("cuda", target)
        ad, xd = a.to(dev).requires_grad_(True), x.to(dev).requires_grad_(True)
        y = btp(ad, xd, output_dtype=torch.bfloat16)
        y.backward(dy.to(dev))
        torch.cuda.synchronize(dev)
        assert y.device == dev and xd.grad.device == dev
        assert O.rel_l2(y.float().cpu(), y_w) <= 1e-2
        assert O.rel_l2(xd.grad.float().cpu(), dx_w) <= 1e-2
        assert O.rel_l2(ad.grad.float().cpu(), dA_w) <= 1e-2
        outs.setdefault(target, []).append((y.detach().cpu(), xd.grad.cpu()))
        assert torch.cuda.current_device() == current  # the call leaves the current device as it found it
    for target in (0, 1):
        assert torch.equal(outs[target][0][0], outs[target][1][0])
    assert torch.equal(outs[0][0][0], outs[1][0][0]) and torch.equal(outs[0][0][1], outs[1][0][1])
    # the no-allocation entry keeps one scratch array per device
    lib = _lib.load()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    ys = []
    for target in (1, 0):
        torch.cuda.set_device(target)
        dev = torch.device("cuda", target)
        ad, xd = a.to(dev), x.to(dev)
        y = torch.empty_like(xd)
        rc = lib.btp_sm100_forward_noalloc(p(ad), p(xd), p(y), B, H, L, 2, 0, 0, ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        assert rc == 0, lib.btp_sm100_last_error().decode()
        # the record went to THIS device's copy of the array: it equals the checkpoint of the ordinary entry point
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        nb = L // 16
        ckpt = torch.empty(B, H, nb, 16, device=dev, dtype=torch.float32)
        y2 = torch.empty_like(xd)
        assert lib.btp_sm100_forward(p(ad), p(xd), p(y2), p(ckpt), B, H, L, 2, 0, 0, stream) == 0
        record = torch.full((B, H, nb, 16), float("nan"), device=dev, dtype=torch.float32)
        assert lib.btp_sm100_noalloc_read_record(p(record), record.numel(), stream) == 0
        torch.cuda.synchronize(dev)
        assert torch.equal(record[:, :, : nb - 1], ckpt[:, :, : nb - 1])
        ys.append(y.cpu())
    assert torch.equal(ys[0], ys[1]) and O.rel_l2(ys[0].float(), y_w) <= 1e-2
    # a layer on the second device while the first one is current
    torch.cuda.set_device(0)
    layer = Phalanx(dim=128, length=64, dtype=torch.bfloat16).to("cuda:1")
    u = torch.randn(2, 64, 128, device="cuda:1", dtype=torch.bfloat16, requires_grad=True)
    layer(u).sum().backward()
    assert u.grad.device == torch.device("cuda", 1) and torch.isfinite(u.grad).all()
    _lib.device_status()
