"""The measured tiling choice (``natten_mlx_b200.tune.tune_fused`` over ``natten_b200_plan_hint``):
whatever it pins, results stay those of the oracle; hints can be set, refused and released."""

from __future__ import annotations

import ctypes

import pytest
import torch

import natten_oracle as oracle

import natten_mlx_b200 as nb
from natten_mlx_b200 import _lib
from natten_mlx_b200._core import cuda as backend

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(shape, seed):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)


def test_tuned_plans_keep_parity():
    shape, ks, dl, ca = (2, 40, 36, 2, 32), (7, 5), (1, 2), (False, False)
    q, k, v, cot = (_rand(shape, s) for s in (1, 2, 3, 4))
    fn = lambda a, b, c: oracle.na(a, b, c, ks, 1, dl, ca, return_lse=True)
    (o_ref, l_ref), g_ref = oracle.grads(fn, [q.float(), k.float(), v.float()], (cot.float(), torch.zeros(shape[:-1])))
    qd, kd, vd, cd = (t.to(DEV) for t in (q, k, v, cot))
    res = nb.tune.tune_fused(qd, kd, vd, ks, dilation=dl, is_causal=ca, max_cols=(0, 96, 48), repeats=1)
    assert set(res) == {"fna_fwd_sm100", "fna_bwd_dq_sm100", "fna_bwd_dkv_sm100"}
    one = (1, 1)
    out, lse = backend.fused_forward(qd, kd, vd, ks, one, dl, ca, None, path="tcgen05")
    dq, dk, dv, _, _ = backend.fused_backward(qd, kd, vd, out, lse, cd, None, ks, one, dl, ca, None, path="tcgen05")
    assert _lib.kernel_status() == 0
    rel = lambda a, b: float((a.float().cpu() - b).abs().max() / b.abs().max())
    assert rel(out, o_ref) < 2e-2 and rel(lse, l_ref) < 2e-2
    for a, b in zip((dq, dk, dv), g_ref):
        assert rel(a, b) < 2e-2


def test_plan_hint_set_refuse_release():
    lib = _lib.load()
    g = _lib.make_geom(2, 1, 2, 2, 32, _lib.BF16, [32, 32], [5, 5], [1, 1], [1, 1], [0, 0], 32 ** -0.5)
    auto = _lib.describe_plan(g)
    tile = (ctypes.c_int32 * 3)(8, 16, 0)
    assert lib.natten_b200_plan_hint(g, 0, tile, 64) == _lib.OK
    pinned = _lib.describe_plan(g).split(" | ")[0]
    assert pinned.startswith("tile 1x8x16")
    bad = (ctypes.c_int32 * 3)(3, 5, 0)                       # not a tile the kernels can take
    assert lib.natten_b200_plan_hint(g, 0, bad, 0) == _lib.EINVAL and "plan_hint" in _lib.last_error()
    assert lib.natten_b200_plan_hint(g, 3, None, 0) == _lib.EINVAL
    assert lib.natten_b200_plan_hint(g, 0, None, 0) == _lib.OK
    assert _lib.describe_plan(g) == auto


def test_tuned_plans_of_a_variable_size_batch_with_extra_tokens_keep_parity():
    sizes = [(24, 20), (16, 28)]
    q = _rand((2, 24, 28, 4, 32), 11)
    k, v = _rand((2, 24, 28, 2, 32), 12), _rand((2, 24, 28, 2, 32), 13)
    ak, av = _rand((2, 6, 2, 32), 14), _rand((2, 6, 2, 32), 15)
    cot = _rand((2, 24, 28, 4, 32), 16)
    ks, dl = (5, 3), (1, 2)
    ref = lambda *t: oracle.na_varlen(t[0], t[1], t[2], sizes, ks, dl, additional_keys=t[3], additional_values=t[4])
    o_ref, g_ref = oracle.grads(ref, [t.float() for t in (q, k, v, ak, av)], cot.float())
    dev = [t.to(DEV) for t in (q, k, v, ak, av)]
    st = torch.tensor(sizes, dtype=torch.int32, device=DEV)
    res = nb.tune.tune_fused(dev[0], dev[1], dev[2], ks, dilation=dl, max_cols=(0, 96, 48), repeats=1, sizes=st,
                             host_sizes=sizes, additional_keys=dev[3], additional_values=dev[4])
    assert set(res) == {"fna_fwd_sm100", "fna_bwd_dq_sm100", "fna_bwd_dkv_sm100"}
    leaves = [t.requires_grad_(True) for t in dev]
    out = nb.na2d_varlen(*leaves[:3], st, ks, dl, additional_keys=leaves[3], additional_values=leaves[4], host_sizes=sizes)
    assert _lib.last_path() == "tcgen05"
    grads = torch.autograd.grad(out, leaves, cot.to(DEV))
    assert _lib.kernel_status() == 0
    rel = lambda a, b: float((a.detach().float().cpu() - b).abs().max() / b.abs().max())
    assert rel(out, o_ref) < 2e-2
    for a, b in zip(grads, g_ref):
        assert rel(a, b) < 2e-2
