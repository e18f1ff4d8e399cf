"""The reference's tests/btp/test_operators.py against the `btp()` wrapper here: shapes, default output dtype,
batch / length / head sweeps, gradient flow, repeatability, minimum and large sizes, every accepted `wpb`.

One difference is deliberate: the reference's tests pass a coefficient tensor of shape [H, 2, 32], which its
wrapper never checks (spear/ops/btp/interface.py:136-139) although the kernel reads B*H*L coefficients.  Here the
coefficients have the shape the kernel reads, [B, H, L], and anything else is an error."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, H, L, grad=False):
    coeff = torch.rand(B, H, L, device="cuda").bfloat16().requires_grad_(grad)
    x = torch.randn(B, H, 16, L, dtype=torch.bfloat16, device="cuda").requires_grad_(grad)
    return coeff, x


@pytest.mark.parametrize("B,H,L", [(1, 4, 256), (2, 8, 512), (4, 16, 1024), (1, 1, 16), (8, 32, 2048)])
def test_btp_forward_basic(B, H, L):
    from spear_b200.ops.btp import btp

    coeff, x = _inputs(B, H, L)
    y = btp(coeff, x)
    assert y.shape == x.shape and y.dtype == torch.float32 and y.device == x.device
    assert torch.isfinite(y).all()


@pytest.mark.parametrize("B", [1, 2, 4, 8])
@pytest.mark.parametrize("L", [64, 128, 256, 512, 1024])
def test_btp_forward_batch_and_length_sweep(B, L):
    from spear_b200.ops.btp import btp

    coeff, x = _inputs(B, 8, L)
    assert btp(coeff, x, output_dtype=torch.bfloat16).shape == x.shape


@pytest.mark.parametrize("H", [4, 8, 16, 32])
def test_btp_forward_different_head_counts(H):
    from spear_b200.ops.btp import btp

    coeff, x = _inputs(2, H, 512)
    assert btp(coeff, x).shape == x.shape


def test_btp_gradient_flow_and_memory():
    from spear_b200.ops.btp import btp

    coeff, x = _inputs(4, 16, 1024, grad=True)
    btp(coeff, x).sum().backward()
    assert coeff.grad is not None and coeff.grad.shape == coeff.shape
    assert x.grad is not None and x.grad.shape == x.shape and x.grad.dtype == x.dtype
    assert torch.isfinite(coeff.grad).all() and torch.isfinite(x.grad).all()


def test_btp_same_input_same_output():
    from spear_b200.ops.btp import btp

    coeff, x = _inputs(2, 8, 512)
    assert torch.equal(btp(coeff, x), btp(coeff, x))


def test_btp_different_wpb_values():
    from spear_b200.ops.btp import btp

    coeff, x = _inputs(2, 8, 512)
    ref = btp(coeff, x)
    for wpb in (4, 8, 16, 32):  # accepted for compatibility; the result does not depend on it
        assert torch.equal(btp(coeff, x, wpb=wpb), ref)
    with pytest.raises((AssertionError, RuntimeError)):
        btp(coeff, x, wpb=5)


def test_btp_rejects_the_coefficient_shape_the_reference_tests_pass():
    from spear_b200.ops.btp import btp

    x = torch.randn(2, 8, 16, 512, dtype=torch.bfloat16, device="cuda")
    with pytest.raises((ValueError, RuntimeError), match="coeff"):
        btp(torch.randn(8, 2, 32, dtype=torch.bfloat16, device="cuda"), x)
