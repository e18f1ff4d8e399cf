"""GPU side of the reference's tests/phalanx/test_layers.py for the layer mirror: shapes, dtypes and devices
are preserved, any batch size works, key/value head sharing works, gradients reach every parameter."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,L,dim", [(1, 64, 128), (2, 128, 256), (4, 256, 512)])
def test_phalanx_forward_shape_preservation(B, L, dim):
    from spear_b200.nn.phalanx import Phalanx

    layer = Phalanx(dim=dim, length=L, dtype=torch.bfloat16).cuda()
    x = torch.randn(B, L, dim, dtype=torch.bfloat16, device="cuda")
    y = layer(x)
    assert y.shape == x.shape and y.dtype == x.dtype and y.device == x.device
    assert torch.isfinite(y).all()


def test_phalanx_forward_different_batch_sizes_and_kv_heads():
    from spear_b200.nn.phalanx import Phalanx

    for kv_heads in (None, 4):
        layer = Phalanx(dim=256, length=128, dtype=torch.bfloat16, kv_heads=kv_heads).cuda()
        for B in (1, 2, 4, 8):
            x = torch.randn(B, 128, 256, dtype=torch.bfloat16, device="cuda")
            assert layer(x).shape == x.shape


@pytest.mark.parametrize("fused", [True, False])
def test_phalanx_gradient_flow(fused):
    from spear_b200.nn.phalanx import Phalanx

    layer = Phalanx(dim=256, length=128, dtype=torch.bfloat16).cuda()
    layer.fused_gating = fused
    x = torch.randn(2, 128, 256, dtype=torch.bfloat16, device="cuda", requires_grad=True)
    layer(x).sum().backward()
    assert x.grad is not None and x.grad.shape == x.shape and torch.isfinite(x.grad).all()
    for name, p in layer.named_parameters():
        assert p.grad is not None, name
        assert torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0, name


def test_layers_with_identical_weights_agree():
    """Two layers built under the same seed give the same output (test_layers.py:301-321)."""
    from spear_b200.nn.phalanx import Phalanx

    x = torch.randn(2, 128, 256, dtype=torch.bfloat16, device="cuda")
    outs = []
    for _ in range(2):
        torch.manual_seed(42)
        outs.append(Phalanx(dim=256, length=128, dtype=torch.bfloat16).cuda()(x))
    assert torch.equal(outs[0], outs[1])
