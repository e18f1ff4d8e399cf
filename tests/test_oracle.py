"""The CPU oracle against the golden vectors produced by the reference's own
PyTorch path (tests/golden/make_golden.py).  No GPU needed."""

from __future__ import annotations

import os
import sys

import pytest
import torch

import btp_oracle as O
from conftest import OP_CASES, load_golden


def _close(got, want, rtol, atol, what):
    assert got.shape == want.shape, what
    assert torch.allclose(got.double(), want.double(), rtol=rtol, atol=atol), (
        f"{what}: max abs diff {(got.double() - want.double()).abs().max().item():.3e}"
    )


@pytest.mark.parametrize("case", OP_CASES)
def test_forward_fp64_product_matches_reference(case):
    g = load_golden(case)
    y = O.btp_forward(g["a"].double(), g["x"].double(), 2, "product")
    _close(y, g["y_ref64"], 1e-12, 1e-13, "y fp64")


@pytest.mark.parametrize("case", [c for c in OP_CASES if c != "op_zeros_ones"])
def test_forward_fp32_log_matches_reference(case):
    g = load_golden(case)
    y = O.btp_forward(g["a"], g["x"], 2, "log")
    # same algorithm, same dtype, same summation order: agreement to rounding
    _close(y, g["y_log32"], 2e-6, 2e-6, "y fp32 log")


@pytest.mark.parametrize("case", OP_CASES)
def test_forward_fp32_cumprod_matches_reference(case):
    g = load_golden(case)
    y = O.btp_forward(g["a"], g["x"], 2, "cumprod")
    _close(y, g["y_lin32"], 2e-6, 2e-6, "y fp32 linear")


@pytest.mark.parametrize("case", OP_CASES)
def test_backward_closed_form_matches_reference_autograd_fp64(case):
    g = load_golden(case)
    dA, dx = O.btp_backward(g["a"].double(), g["x"].double(), g["dy"].double(), 2, "product")
    _close(dx, g["dx_ref64"], 1e-11, 1e-12, "dx fp64")
    _close(dA, g["dA_ref64"], 1e-10, 1e-11, "dA fp64")


@pytest.mark.parametrize("case", [c for c in OP_CASES if c != "op_zeros_ones"])
def test_backward_closed_form_fp32_log(case):
    g = load_golden(case)
    dA, dx = O.btp_backward(g["a"], g["x"], g["dy"], 2, "log")
    assert O.rel_l2(dx, g["dx_log32"]) < 1e-6
    assert O.rel_l2(dA, g["dA_log32"]) < 1e-5
    assert O.rel_l2(dA, g["dA_ref64"]) < 1e-5


@pytest.mark.parametrize("case", OP_CASES)
def test_k1_local_pass_only(case):
    g = load_golden(case)
    y = O.btp_forward(g["a"].double(), g["x"].double(), 1, "product")
    _close(y, g["y_k1_ref64"], 1e-12, 1e-13, "y k=1")
    dA, dx = O.btp_backward(g["a"].double(), g["x"].double(), g["dy"].double(), 1, "product")
    _close(dx, g["dx_k1_ref64"], 1e-11, 1e-12, "dx k=1")
    _close(dA, g["dA_k1_ref64"], 1e-10, 1e-11, "dA k=1")


def test_autograd_helper_agrees_with_closed_form():
    g = load_golden("op_basic")
    y, dA, dx = O.btp_forward_backward_autograd(g["a"].double(), g["x"].double(), g["dy"].double(), "product")
    dA2, dx2 = O.btp_backward(g["a"].double(), g["x"].double(), g["dy"].double(), 2, "product")
    _close(dA, dA2, 1e-10, 1e-11, "dA")
    _close(dx, dx2, 1e-11, 1e-12, "dx")
    _close(y, g["y_ref64"], 1e-12, 1e-13, "y")


def test_one_hop_only():
    """Changing block 0 changes block 1 and leaves block 2 bit-identical: the op is
    a sliding window, not a full recurrence (reference.py:123-136)."""
    g = load_golden("op_basic")
    a, x = g["a"], g["x"]
    y0 = O.btp_forward(a, x)
    x2 = x.clone()
    x2[..., :16] += 1.0
    y1 = O.btp_forward(a, x2)
    assert not torch.equal(y0[..., 16:32], y1[..., 16:32])
    assert torch.equal(y0[..., 32:], y1[..., 32:])


def test_shape_validation():
    a = torch.rand(1, 2, 24)
    x = torch.rand(1, 2, 16, 24)
    with pytest.raises(ValueError):
        O.btp_forward(a, x)
    with pytest.raises(ValueError):
        O.btp_forward(torch.rand(1, 3, 32), torch.rand(1, 2, 16, 32))


# ------------------------------------------------------------------ the layer's data flow around the op
@pytest.mark.parametrize("case,kv_heads", [("layer_basic", None), ("layer_kv2", 2)])
def test_oracle_layer_matches_reference_layer(case, kv_heads):
    g = load_golden(case)
    state = {k[2:]: v for k, v in g.items() if k.startswith("w:")}
    out = O.phalanx_forward(state, g["u"], kv_heads=kv_heads)
    assert torch.allclose(out, g["out"], rtol=1e-4, atol=1e-5)


def cfg0_tensors():
    """Weights and inputs of the reference's CPU-runnable configuration (dim 512, length 128, batch 8, float32),
    regenerated from the seeds tests/golden/make_golden.py used and verified against the stored checksums."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    from make_golden import CFG0, cfg0_inputs
    from spear_b200.nn.phalanx import Phalanx

    g = load_golden("layer_cfg0")
    torch.manual_seed(CFG0["weight_seed"])
    layer = Phalanx(dim=CFG0["dim"], length=CFG0["length"], dtype=torch.float32)
    u, dout = cfg0_inputs()
    chk = lambda t: torch.tensor([t.double().sum().item(), t.double().abs().sum().item()], dtype=torch.float64)
    for name, t in layer.state_dict().items():
        assert torch.allclose(chk(t), g["wsum:" + name], rtol=1e-12, atol=0), f"seeded init of {name} differs from the fixture's"
    assert torch.allclose(chk(u), g["u_checksum"], rtol=1e-12, atol=0)
    assert torch.allclose(chk(dout), g["dout_checksum"], rtol=1e-12, atol=0)
    return g, layer, u, dout, CFG0["stride"]


def test_oracle_layer_matches_reference_at_its_cpu_configuration():
    g, layer, u, _, st = cfg0_tensors()
    out = O.phalanx_forward(layer.state_dict(), u)
    assert torch.allclose(out[:, ::st, ::st], g["out_sample"], rtol=1e-4, atol=1e-5)
    assert abs(out.double().norm().item() / g["out_norm"].item() - 1.0) < 1e-5
