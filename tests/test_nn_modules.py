"""torch modules (``natten_mlx_b200.nn``): construction and validation run without a GPU;
the GPU cases compare a module's output and parameter gradients with the same
computation written out against the CPU oracle (projection → oracle operator →
projection), for the configurations the reference's module tests cover
(tests/test_na2d.py:8-57, tests/test_nn_module_grad.py:20-380): stride, causal,
dilation, no qkv bias, custom scale, attention dropout (split path), GQA / MQA,
per-sample sizes."""

from __future__ import annotations

import pytest
import torch

import natten_oracle as oracle

from natten_mlx_b200.nn import NeighborhoodAttention1D, NeighborhoodAttention2D, NeighborhoodAttention3D

MODS = {1: NeighborhoodAttention1D, 2: NeighborhoodAttention2D, 3: NeighborhoodAttention3D}


def test_construction_and_parameter_shapes():
    m = NeighborhoodAttention2D(embed_dim=12, num_heads=4, kernel_size=(3, 5), dilation=2)
    assert m.head_dim == 3 and m.kernel_size == (3, 5) and m.dilation == (2, 2) and m.is_causal == (False, False)
    assert m.qkv.weight.shape == (36, 12) and m.q_proj is None and m.proj.weight.shape == (12, 12)
    g = NeighborhoodAttention1D(embed_dim=16, num_heads=4, kernel_size=3, num_kv_heads=2, qkv_bias=False)
    assert g.qkv is None and g.q_proj.weight.shape == (16, 16) and g.kv_proj.weight.shape == (16, 16)
    assert g.q_proj.bias is None and g.scale == 4 ** -0.5
    assert NeighborhoodAttention3D(8, 2, 3, qk_scale=0.3).scale == 0.3


@pytest.mark.parametrize("kwargs,match", [
    (dict(embed_dim=0, num_heads=1, kernel_size=3), "embed_dim"),
    (dict(embed_dim=8, num_heads=0, kernel_size=3), "num_heads"),
    (dict(embed_dim=10, num_heads=4, kernel_size=3), "divisible"),
    (dict(embed_dim=12, num_heads=4, kernel_size=3, num_kv_heads=3), "divisible"),
])
def test_construction_errors(kwargs, match):
    with pytest.raises(ValueError, match=match):
        NeighborhoodAttention1D(**kwargs)


def test_input_shape_errors():
    m = NeighborhoodAttention1D(8, 2, 3)
    with pytest.raises(ValueError, match=r"\[B, L, C\]"):
        m(torch.zeros(2, 5, 5, 8))
    with pytest.raises(ValueError, match="embed_dim"):
        m(torch.zeros(2, 5, 6))


def _reference(m, x, sizes=None):
    """The module's computation with the oracle in place of the CUDA operator (float32, CPU)."""
    w = {k: v.detach().cpu().double().float().requires_grad_(True) for k, v in m.named_parameters()}
    xc = x.detach().cpu().requires_grad_(True)
    lin = lambda name, t: torch.nn.functional.linear(t, w[name + ".weight"], w.get(name + ".bias"))
    lead = tuple(xc.shape[:-1])
    if m.qkv is not None:
        qkv = lin("qkv", xc).view(*lead, 3, m.num_heads, m.head_dim)
        q, k, v = qkv.select(-3, 0), qkv.select(-3, 1), qkv.select(-3, 2)
    else:
        q = lin("q_proj", xc).view(*lead, m.num_heads, m.head_dim)
        kv = lin("kv_proj", xc).view(*lead, 2, m.num_kv_heads, m.head_dim)
        k, v = kv.select(-3, 0), kv.select(-3, 1)
    if sizes is None:
        o = oracle.na(q, k, v, m.kernel_size, m.stride, m.dilation, m.is_causal, scale=m.scale)
    else:
        o = oracle.na_varlen(q, k, v, sizes, m.kernel_size, m.dilation, scale=m.scale)
    y = lin("proj", o.reshape(*o.shape[:-2], m.embed_dim))
    return y, xc, w


CASES = [
    # rank, input shape, module arguments
    (1, (2, 19, 12), dict(embed_dim=12, num_heads=4, kernel_size=5)),
    (1, (2, 19, 12), dict(embed_dim=12, num_heads=4, kernel_size=5, stride=2, is_causal=True, qkv_bias=False)),
    (1, (2, 24, 16), dict(embed_dim=16, num_heads=4, kernel_size=3, dilation=3, num_kv_heads=2, qk_scale=0.37)),
    (1, (2, 24, 16), dict(embed_dim=16, num_heads=4, kernel_size=3, num_kv_heads=1)),
    (2, (2, 7, 5, 12), dict(embed_dim=12, num_heads=4, kernel_size=(3, 3))),
    (2, (2, 8, 9, 12), dict(embed_dim=12, num_heads=4, kernel_size=(3, 5), stride=(2, 1), is_causal=(True, False),
                            attn_drop=0.25)),
    (2, (1, 10, 8, 16), dict(embed_dim=16, num_heads=4, kernel_size=3, dilation=2, num_kv_heads=2)),
    (3, (1, 5, 6, 7, 8), dict(embed_dim=8, num_heads=2, kernel_size=(3, 3, 5), is_causal=(True, False, False))),
    (3, (1, 4, 6, 6, 8), dict(embed_dim=8, num_heads=4, kernel_size=3, stride=(1, 2, 2), num_kv_heads=2)),
]


@pytest.mark.gpu
@pytest.mark.parametrize("rank,shape,kwargs", CASES)
def test_module_matches_oracle_composition(rank, shape, kwargs):
    torch.manual_seed(11)
    m = MODS[rank](**kwargs).to("cuda").eval()          # eval: dropout inactive, the split path must equal the fused one
    x = torch.randn(shape, generator=torch.Generator().manual_seed(3)).to("cuda").requires_grad_(True)
    y = m(x)
    y_ref, x_ref, w_ref = _reference(m, x)
    assert y.shape == y_ref.shape
    assert torch.allclose(y.detach().cpu(), y_ref.detach(), atol=2e-4, rtol=2e-4)
    cot = torch.randn(y_ref.shape, generator=torch.Generator().manual_seed(4))
    y.backward(cot.to("cuda"))
    y_ref.backward(cot)
    assert torch.allclose(x.grad.cpu(), x_ref.grad, atol=5e-4, rtol=5e-4)
    for name, p in m.named_parameters():
        assert p.grad is not None, name
        assert torch.allclose(p.grad.cpu(), w_ref[name].grad, atol=1e-3, rtol=1e-3), name


@pytest.mark.gpu
def test_module_training_dropout_runs_split_path():
    m = NeighborhoodAttention2D(12, 4, 3, attn_drop=0.5, proj_drop=0.1).to("cuda").train()
    y = m(torch.randn(2, 7, 5, 12, device="cuda"))
    assert y.shape == (2, 7, 5, 12) and torch.isfinite(y).all()


@pytest.mark.gpu
def test_module_with_per_sample_sizes():
    m = NeighborhoodAttention2D(8, 2, 3).to("cuda").eval()
    x = torch.randn(3, 9, 10, 8, generator=torch.Generator().manual_seed(8)).to("cuda")
    sizes = torch.tensor([[9, 10], [5, 7], [3, 4]], dtype=torch.int32)
    y = m(x, sizes.to("cuda"))
    y_ref, _, _ = _reference(m, x, sizes)
    assert torch.allclose(y.detach().cpu(), y_ref.detach(), atol=2e-4, rtol=2e-4)
