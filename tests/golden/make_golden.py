"""Generate the golden fixtures in this folder from the reference's own PyTorch path.

Run once, in a container where the reference checkout is mounted:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/spear

It imports spear/ops/btp/reference.py (by file path) and the Phalanx layer
(with a stand-in module registered for the compiled extension, which the
pure-PyTorch methods never call), evaluates them on seeded inputs and writes
small .npz files.  The fixtures travel with the repository; the reference
checkout does not, so no test reads it at run time.
"""

from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_reference_math(root: str):
    path = os.path.join(root, "spear", "ops", "btp", "reference.py")
    spec = importlib.util.spec_from_file_location("_spear_btp_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _bf16_grid(t: torch.Tensor) -> torch.Tensor:
    """Round to values representable in bf16, keep float32 storage."""
    return t.to(torch.bfloat16).to(torch.float32)


def _grads(fn, a, x, dy):
    a = a.clone().requires_grad_(True)
    x = x.clone().requires_grad_(True)
    y = fn(a, x)
    y.backward(dy.to(y.dtype))
    return y.detach(), a.grad.detach(), x.grad.detach()


def _op_case(R, name, a, x, dy, *, zero_safe=False):
    """One op-level fixture: outputs of the log/fp32, explicit-product/fp64 and
    linear-space/fp32 reference paths plus their autograd gradients."""
    out = {"a": a.numpy(), "x": x.numpy(), "dy": dy.numpy()}
    y64, dA64, dx64 = _grads(R.block_two_pass_ref, a.double(), x.double(), dy.double())
    out.update(y_ref64=y64.numpy(), dA_ref64=dA64.numpy(), dx_ref64=dx64.numpy())
    ylin, dAlin, dxlin = _grads(R.block_two_pass_linspace, a, x, dy)
    out.update(y_lin32=ylin.numpy(), dA_lin32=dAlin.numpy(), dx_lin32=dxlin.numpy())
    if not zero_safe:  # log(0) makes the log path's autograd NaN
        ylog, dAlog, dxlog = _grads(R.block_two_pass_log, a, x, dy)
        out.update(y_log32=ylog.numpy(), dA_log32=dAlog.numpy(), dx_log32=dxlog.numpy())
    # k = 1 (local pass only): every 16-token block as its own sequence
    B, H, D, L = x.shape
    nb = L // 16
    a1 = a.reshape(B, H * nb, 16)
    x1 = x.reshape(B, H, D, nb, 16).permute(0, 1, 3, 2, 4).reshape(B, H * nb, D, 16)
    dy1 = dy.reshape(B, H, D, nb, 16).permute(0, 1, 3, 2, 4).reshape(B, H * nb, D, 16)
    yk1, dAk1, dxk1 = _grads(R.block_two_pass_ref, a1.double(), x1.double(), dy1.double())
    unblock = lambda t: t.reshape(B, H, nb, D, 16).permute(0, 1, 3, 2, 4).reshape(B, H, D, L)
    out.update(y_k1_ref64=unblock(yk1).numpy(), dx_k1_ref64=unblock(dxk1).numpy(),
               dA_k1_ref64=dAk1.reshape(B, H, L).numpy())
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
    print(f"wrote {name}.npz", {k: v.shape for k, v in out.items() if k in ('a', 'x')})


def make_op_fixtures(R):
    g = torch.Generator().manual_seed(123)

    def sample(B, H, L, coeff_std=1.0, x_std=1.0):
        x = _bf16_grid(torch.randn(B, H, 16, L, generator=g) * x_std)
        a = _bf16_grid(torch.sigmoid(torch.randn(B, H, L, generator=g) * coeff_std))
        dy = _bf16_grid(torch.randn(B, H, 16, L, generator=g))
        return a, x, dy

    _op_case(R, "op_basic", *sample(2, 3, 64))
    _op_case(R, "op_single_block", *sample(1, 2, 16))
    _op_case(R, "op_two_blocks", *sample(1, 1, 32))
    _op_case(R, "op_stress", *sample(2, 2, 128, coeff_std=4.0, x_std=1.5))
    _op_case(R, "op_ragged_chunk", *sample(1, 2, 208))  # 13 blocks: not a multiple of 8 blocks

    # exact zeros and exact ones among the coefficients
    a, x, dy = sample(1, 2, 64)
    a[0, 0, 5] = 0.0
    a[0, 0, 16] = 0.0  # first token of a block: kills the incoming carry
    a[0, 0, 47] = 0.0  # last token of a block
    a[0, 1, 20:40] = 1.0
    a[0, 1, 0] = 0.0
    _op_case(R, "op_zeros_ones", a, x, dy, zero_safe=True)

    # near-unit decay given in float32 (not representable in bf16)
    a, x, dy = sample(1, 2, 256)
    a = torch.exp(-1e-3 * torch.rand(1, 2, 256, generator=g))
    x = _bf16_grid(torch.randn(1, 2, 16, 256, generator=g) * 0.25)
    _op_case(R, "op_near_unit_f32", a, x, dy)


def make_layer_fixture(root: str):
    sys.path.insert(0, root)
    sys.modules.setdefault("spear._btp", types.ModuleType("spear._btp"))
    from spear.nn.phalanx import Phalanx  # noqa: WPS433

    for name, kv_heads in (("layer_basic", None), ("layer_kv2", 2)):
        torch.manual_seed(987)
        layer = Phalanx(dim=64, length=48, method="pytorch", dtype=torch.float32, kv_heads=kv_heads)
        layer.param.compute_dtype = torch.float32  # the fp32 layer only runs with this override
        g = torch.Generator().manual_seed(789)
        u = torch.randn(2, 48, 64, generator=g)
        dout = torch.randn(2, 48, 64, generator=g)
        u_in = u.clone().requires_grad_(True)
        out = layer(u_in)
        out.backward(dout)
        data = {"u": u.numpy(), "dout": dout.numpy(), "out": out.detach().numpy(), "du": u_in.grad.numpy()}
        for k, v in layer.state_dict().items():
            data["w:" + k] = v.numpy()
        for k, p in layer.named_parameters():
            data["g:" + k] = p.grad.numpy()
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **data)
        print(f"wrote {name}.npz")


CFG0 = dict(dim=512, length=128, batch=8, weight_seed=2024, input_seed=4048, stride=8)


def cfg0_inputs():
    """Inputs of the `dim=512, length=128, batch=8, fp32` layer case, regenerated from seeds by the test."""
    g = torch.Generator().manual_seed(CFG0["input_seed"])
    u = torch.randn(CFG0["batch"], CFG0["length"], CFG0["dim"], generator=g)
    dout = torch.randn(CFG0["batch"], CFG0["length"], CFG0["dim"], generator=g)
    return u, dout


def make_cfg0_fixture(root: str):
    """The reference's own CPU-runnable configuration: Phalanx forward (and backward) in float32 through its
    PyTorch path.  Weights and inputs come from seeds, so the fixture only keeps checksums of them (the test
    refuses to run if its regenerated tensors differ) and a strided sample of the outputs with their norms."""
    sys.path.insert(0, root)
    sys.modules.setdefault("spear._btp", types.ModuleType("spear._btp"))
    from spear.nn.phalanx import Phalanx  # noqa: WPS433

    torch.manual_seed(CFG0["weight_seed"])
    layer = Phalanx(dim=CFG0["dim"], length=CFG0["length"], method="pytorch", dtype=torch.float32)
    layer.param.compute_dtype = torch.float32
    u, dout = cfg0_inputs()
    u_in = u.clone().requires_grad_(True)
    out = layer(u_in)
    out.backward(dout)
    st = CFG0["stride"]
    data = {"out_sample": out.detach()[:, ::st, ::st].numpy(), "du_sample": u_in.grad[:, ::st, ::st].numpy(),
            "out_norm": np.array(out.detach().double().norm().item()), "du_norm": np.array(u_in.grad.double().norm().item()),
            "u_checksum": np.array([u.double().sum().item(), u.double().abs().sum().item()]),
            "dout_checksum": np.array([dout.double().sum().item(), dout.double().abs().sum().item()])}
    for k, v in layer.state_dict().items():
        data["wsum:" + k] = np.array([v.double().sum().item(), v.double().abs().sum().item()])
    for k, p in layer.named_parameters():
        data["gnorm:" + k] = np.array(p.grad.double().norm().item())
    np.savez_compressed(os.path.join(HERE, "layer_cfg0.npz"), **data)
    print("wrote layer_cfg0.npz")


def make_inference_fixture(root: str):
    """Outputs of the reference's prefill + decode helpers (spear/nn/phalanx/inference.py), float32 on CPU."""
    sys.path.insert(0, root)
    sys.modules.setdefault("spear._btp", types.ModuleType("spear._btp"))
    from spear.nn.phalanx.inference import parallel_jagged, step_jagged  # noqa: WPS433

    g = torch.Generator().manual_seed(4321)
    data = {}
    for L in (40, 64, 7):
        B, H, D, steps = 2, 3, 16, 20
        total = L + steps
        A = _bf16_grid(torch.sigmoid(torch.randn(B, H, total, generator=g)))
        X = _bf16_grid(torch.randn(B, H, D, total, generator=g))
        C = _bf16_grid(torch.randn(B, H, D, total, generator=g))
        V = _bf16_grid(torch.randn(B, H, D, total, generator=g))
        Y, st = parallel_jagged(A[..., :L], X[..., :L], C[..., :L], V[..., :L], block_len=16)
        ys = []
        for t in range(L, total):
            y_t, st = step_jagged(A[..., t], X[..., t], C[..., t], V[..., t], st)
            ys.append(y_t)
        pre = f"L{L}:"
        data.update({pre + "A": A.numpy(), pre + "X": X.numpy(), pre + "C": C.numpy(), pre + "V": V.numpy(),
                     pre + "Y": Y.numpy(), pre + "Ydec": torch.stack(ys, dim=-1).numpy()})
        _, st0 = parallel_jagged(A[..., :L], X[..., :L], C[..., :L], V[..., :L], block_len=16)
        data.update({pre + "h_loc": st0.h_loc.numpy(), pre + "r_pref": st0.r_pref.numpy(),
                     pre + "c_prev_loc": st0.c_prev_loc.numpy(), pre + "i": np.array(st0.i)})
    np.savez_compressed(os.path.join(HERE, "inference.npz"), **data)
    print("wrote inference.npz")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    torch.set_num_threads(4)
    make_op_fixtures(_load_reference_math(args.reference))
    make_layer_fixture(args.reference)
    make_cfg0_fixture(args.reference)
    make_inference_fixture(args.reference)
