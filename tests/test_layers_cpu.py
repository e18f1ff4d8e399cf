"""Host-side behaviour of the layer mirror (KVRepeat, SigmoidA, Phalanx), after the reference's own
tests/phalanx/test_layers.py: construction, attribute names, argument errors, tensor shapes of the projection
stage, parameter names, state-dict round trip.  Everything here is module plumbing and runs on CPU; the
recurrence itself has no CPU path and is only reached by the GPU tests."""

from __future__ import annotations

import pytest
import torch

from spear_b200.nn.phalanx import KVRepeat, Phalanx, SigmoidA


# ------------------------------------------------------------------ KVRepeat (test_layers.py:25-84)
def test_kv_repeat_creation():
    r = KVRepeat(4, 16)
    assert (r.kv_heads, r.total_heads, r.kv_groups, r.enabled) == (4, 16, 4, True)
    assert r.kv_indices.tolist() == [h // 4 for h in range(16)]
    assert "kv_indices" not in r.state_dict()  # non-persistent buffer, as in the reference


def test_kv_repeat_no_grouping():
    r = KVRepeat(16, 16)
    assert (r.kv_groups, r.enabled) == (1, False)
    x = torch.randn(2, 16, 8, 32)
    assert r(x) is x


def test_kv_repeat_invalid_heads():
    with pytest.raises(ValueError, match="must be divisible"):
        KVRepeat(3, 16)


def test_kv_repeat_forward_and_flat_forms():
    r = KVRepeat(4, 16)
    x = torch.randn(2, 4, 8, 32)
    y = r(x)
    assert y.shape == (2, 16, 8, 32) and y.dtype == x.dtype
    for h in range(16):
        assert torch.equal(y[:, h], x[:, h // 4])
    flat = x.reshape(2, 32, 32)
    assert torch.equal(r.expand_and_reshape(flat, 2, 8, 32), y)
    assert torch.equal(r.expand_flat(flat, 8), y.reshape(2, 128, 32))
    assert r.reshape_for_kv(flat, 2, 8, 32).shape == (2, 4, 8, 32)


# ------------------------------------------------------------------ SigmoidA (test_layers.py:85-142)
def test_sigmoid_a_creation():
    s = SigmoidA(256, 16, 16)
    assert (s.dim, s.heads, s.head_dim) == (256, 16, 16)
    assert s.proj_a.bias is not None and s.proj_b.bias is not None and s.proj_c.bias is not None and s.proj_v.bias is None


@pytest.mark.parametrize("kv_heads", [None, 4])
def test_sigmoid_a_forward_axcv_shapes(kv_heads):
    s = SigmoidA(256, 16, 16, dtype=torch.bfloat16, kv_heads=kv_heads)
    assert s.proj_b.out_features == (16 if kv_heads is None else kv_heads) * 16
    x = torch.randn(2, 32, 256, dtype=torch.bfloat16)
    A, X, C, V = s.forward_axcv(x)
    assert A.shape == (2, 16, 32)
    for t in (X, C, V):
        assert t.shape == (2, 16, 16, 32)
    for t in (A, X, C, V):
        assert t.dtype == x.dtype
    assert (A > 0).all() and (A < 1).all()
    packed = s.forward_fused_gates(x)
    assert packed.shape == (2, 3 * 256 + 16, 32)


# ------------------------------------------------------------------ Phalanx (test_layers.py:143-190, 301-364)
def test_phalanx_creation_default():
    layer = Phalanx(dim=256, length=128)
    assert (layer.dim, layer.heads, layer.head_dim, layer.method, layer.k) == (256, 16, 16, "default", 2)
    assert layer.kv_heads == 16
    assert list(layer.state_dict()) == [
        "param.proj_a.weight", "param.proj_a.bias", "param.proj_b.weight", "param.proj_b.bias",
        "param.proj_c.weight", "param.proj_c.bias", "param.proj_v.weight", "proj_out.weight",
    ]


def test_phalanx_length_is_rounded_up_to_a_block():
    assert Phalanx(dim=64, length=100).length == 112


def test_phalanx_argument_errors():
    with pytest.raises(ValueError, match="method must be one of"):
        Phalanx(dim=256, method="invalid")
    with pytest.raises(ValueError, match="must be divisible by heads"):
        Phalanx(dim=256, heads=15)
    with pytest.raises(ValueError, match="head_dim must be 16"):
        Phalanx(dim=256, heads=8)
    with pytest.raises(ValueError, match="must be divisible by 16"):
        Phalanx(dim=250)
    for method in ("pytorch", "pytorch_linspace"):  # the reference's CPU paths are not shipped
        with pytest.raises(NotImplementedError):
            Phalanx(dim=256, method=method)


def test_phalanx_manual_seed_gives_identical_layers():
    torch.manual_seed(42)
    a = Phalanx(dim=128, length=64, dtype=torch.bfloat16)
    torch.manual_seed(42)
    b = Phalanx(dim=128, length=64, dtype=torch.bfloat16)
    for (na, pa), (nb, pb) in zip(a.named_parameters(), b.named_parameters()):
        assert na == nb and torch.equal(pa, pb)


def test_layer_state_dict_serialization(tmp_path):
    torch.manual_seed(3)
    a = Phalanx(dim=128, length=64, dtype=torch.bfloat16, kv_heads=4)
    path = tmp_path / "layer.pt"
    torch.save(a.state_dict(), path)
    b = Phalanx(dim=128, length=64, dtype=torch.bfloat16, kv_heads=4)
    b.load_state_dict(torch.load(path))
    for k, v in a.state_dict().items():
        assert torch.equal(v, b.state_dict()[k])
    with pytest.raises(RuntimeError):  # a layer with other key/value sharing has other shapes
        Phalanx(dim=128, length=64, dtype=torch.bfloat16, kv_heads=2).load_state_dict(a.state_dict())


def test_phalanx_forward_needs_a_gpu():
    layer = Phalanx(dim=64, length=32, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        layer(torch.randn(1, 32, 64, dtype=torch.bfloat16))


def test_packed_projections_keep_parameters_and_follow_in_place_updates():
    """The one-GEMM projection path keeps the four weights as row slices of one matrix: same parameters, same
    state_dict, packed buffer follows optimizer steps and load_state_dict, and is rebuilt after `.to()`."""
    from spear_b200.nn.phalanx.swr import _PackedProjections, _WideProjection

    torch.manual_seed(0)
    layer = Phalanx(dim=128, dtype=torch.float64)
    prm = layer.param
    names_before = list(layer.state_dict())
    before = {k: v.clone() for k, v in layer.state_dict().items()}
    params_before = [id(p) for p in layer.parameters()]
    pk = _PackedProjections(prm)
    assert pk.intact(prm) and list(layer.state_dict()) == names_before
    assert [id(p) for p in layer.parameters()] == params_before  # the same Parameter objects
    assert all(torch.equal(v, before[k]) for k, v in layer.state_dict().items())
    u = torch.randn(2, 16, 128, dtype=torch.float64, requires_grad=True)
    args = (prm.proj_b.weight, prm.proj_c.weight, prm.proj_v.weight, prm.proj_a.weight, prm.proj_b.bias, prm.proj_c.bias, prm.proj_a.bias)
    wide = _WideProjection.apply(u, pk.weight, pk.bias, pk.offsets, *args)
    ref = torch.cat([prm.proj_b(u), prm.proj_c(u), prm.proj_v(u), prm.proj_a(u)], -1)
    assert torch.allclose(wide, ref)
    g = torch.randn_like(wide)
    wide.backward(g)
    got = {n: p.grad.clone() for n, p in prm.named_parameters()}
    du = u.grad.clone()
    for p in prm.parameters():
        p.grad = None
    u.grad = None
    ref.backward(g)
    assert all(torch.allclose(p.grad, got[n]) for n, p in prm.named_parameters()) and torch.allclose(u.grad, du)
    torch.optim.SGD(layer.parameters(), lr=0.1).step()  # in place: the packed matrix moves with the parameters
    assert pk.intact(prm) and torch.equal(pk.weight[:128], prm.proj_b.weight) and not torch.equal(pk.weight[:128], before["param.proj_b.weight"])
    layer.load_state_dict(before)
    assert pk.intact(prm) and torch.equal(pk.weight[:128], before["param.proj_b.weight"])
    layer.to(torch.float32)  # fresh storage for every parameter: the link is gone and is noticed
    assert not pk.intact(prm)
