"""The v0.14 call convention (``natten_mlx_b200.compat``): heads-first tensors, un-scaled QK plus
a relative-position-bias table.  The reference pins these relationally
(tests/test_compat_v014.py: QK+RPB equals split QK without scale plus ``rpb[pb_start + k]``);
here they are compared with the CPU oracle's QK+RPB / AV on transposed tensors, forward and
gradients (q, k, rpb / attn, v)."""

from __future__ import annotations

import pytest
import torch

import natten_oracle as oracle

from natten_mlx_b200 import compat


def test_for_version_selects_the_surface():
    assert compat.for_version("0.14.6").__name__.endswith("compat.v014")
    assert compat.for_version("0.13").__name__.endswith("compat.v014")
    modern = compat.for_version("0.17.5")
    assert hasattr(modern, "na2d") and not modern.__name__.endswith("v014")
    with pytest.raises(ValueError, match="version"):
        compat.for_version("latest")


def test_v014_argument_errors():
    v014 = compat.for_version("0.14")
    q = torch.zeros(1, 2, 8, 4)
    with pytest.raises(ValueError, match=r"\[B, H, L, D\]"):
        v014.natten1dqkrpb(q[0], q[0], torch.zeros(2, 5), 3, 1)
    with pytest.raises(ValueError, match="rpb must be"):
        v014.natten1dqkrpb(q, q, torch.zeros(2, 4), 3, 1)
    with pytest.raises(ValueError):
        v014.natten1dqkrpb(q, q, torch.zeros(2, 17), 9, 1)          # kernel larger than the sequence
    with pytest.raises(ValueError, match="divisible"):
        v014.NeighborhoodAttention1D(dim=10, kernel_size=3, num_heads=4)
    m = v014.NeighborhoodAttention2D(dim=8, kernel_size=3, dilation=2, num_heads=2)
    assert m.dim == 8 and m.stride == (1, 1) and m.is_causal == (False, False) and m.num_kv_heads == 2


def _rand(shape, seed):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed))


@pytest.mark.gpu
@pytest.mark.parametrize("length,ks,dl", [(17, 5, 1), (24, 3, 4), (9, 9, 1)])
def test_v014_1d_ops_match_oracle(length, ks, dl):
    v014 = compat.for_version("0.14.6")
    B, H, D = 2, 3, 8
    q, k, v = _rand((B, H, length, D), 1), _rand((B, H, length, D), 2), _rand((B, H, length, D), 3)
    rpb = _rand((H, 2 * ks - 1), 4) * 0.1
    cot = _rand((B, H, length, ks), 5)
    ref = lambda a, b, r: oracle.qk_rpb(a.transpose(1, 2), b.transpose(1, 2), r, ks, dl, 1.0).transpose(1, 2)
    (want,), g_want = oracle.grads(lambda a, b, r: (ref(a, b, r),), [q, k, rpb], (cot,))
    qd, kd, rd = (t.cuda().requires_grad_(True) for t in (q, k, rpb))
    got = v014.natten1dqkrpb(qd, kd, rd, ks, dl)
    fin = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got).cpu(), fin)              # the -inf pattern is exact
    assert torch.allclose(got.detach().cpu()[fin], want[fin], atol=1e-4, rtol=1e-4)
    got.masked_fill(~fin.cuda(), 0.0).mul(cot.cuda().masked_fill(~fin.cuda(), 0.0)).sum().backward()
    for a, b in zip((qd, kd, rd), g_want):
        assert torch.allclose(a.grad.cpu(), b, atol=1e-4, rtol=1e-4)
    attn = torch.softmax(want, dim=-1)
    out_want = oracle.av_fused(attn.transpose(1, 2), v.transpose(1, 2), ks, dl).transpose(1, 2)
    out = v014.natten1dav(attn.cuda(), v.cuda(), ks, dl)
    assert torch.allclose(out.cpu(), out_want, atol=1e-4, rtol=1e-4)


@pytest.mark.gpu
def test_v014_2d_ops_match_oracle():
    v014 = compat.for_version("0.14.6")
    B, H, Hh, Ww, D, ks, dl = 1, 2, 9, 11, 8, 3, 2
    q, k, v = (_rand((B, H, Hh, Ww, D), s) for s in (1, 2, 3))
    rpb = _rand((H, 2 * ks - 1, 2 * ks - 1), 4) * 0.1
    perm, back = (0, 2, 3, 1, 4), (0, 3, 1, 2, 4)
    want = oracle.qk_rpb(q.permute(perm), k.permute(perm), rpb, ks, dl, 1.0).permute(back)
    got = v014.natten2dqkrpb(q.cuda(), k.cuda(), rpb.cuda(), ks, dl).cpu()
    fin = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got), fin)
    assert torch.allclose(got[fin], want[fin], atol=1e-4, rtol=1e-4)
    attn = torch.softmax(want, dim=-1)
    out_want = oracle.av_fused(attn.permute(perm), v.permute(perm), ks, dl).permute(back)
    out = v014.natten2dav(attn.cuda(), v.cuda(), ks, dl).cpu()
    assert torch.allclose(out, out_want, atol=1e-4, rtol=1e-4)
