"""CUDA path against the reference's results (golden fixtures) and the CPU oracle.

Everything here goes through the public API, i.e. through the C ABI of
``libnatten_b200.so``.  Tolerances: index / mask patterns bit-exact; float32
within 1e-4 (max-abs and relative); bf16 / fp16 within 2e-2 of the float32
oracle: relative to the largest reference magnitude, and per element
(|err| <= 5e-2 * (|ref| + rms(ref))); the observed errors of a run are recorded
by ``conftest.assert_lowp``.
"""

from __future__ import annotations

import itertools
import json

import numpy as np
import pytest
import torch

import natten_oracle as oracle
from conftest import assert_lowp, tup
from make_golden import CASES, make_inputs

import natten_mlx_b200 as nb
from natten_mlx_b200 import _lib
from natten_mlx_b200.extras import allin1

pytestmark = pytest.mark.gpu

FP32 = dict(atol=1e-4, rtol=1e-4)
LOWP_REL = 2e-2
DEV = "cuda"


def close32(got, want, name=""):
    got = got.detach().float().cpu().numpy()
    want = want.detach().float().cpu().numpy() if torch.is_tensor(want) else np.asarray(want)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    assert np.array_equal(np.isinf(got), np.isinf(want)), f"{name}: -inf pattern differs"
    fin = np.isfinite(want)
    np.testing.assert_allclose(got[fin], want[fin], err_msg=name, **FP32)


def close_lowp(got, want, name="", rel=LOWP_REL):
    """2e-2 in the max norm, 5e-2 * (|ref| + rms(ref)) per element; observed errors are recorded."""
    assert_lowp(got, want, name, rel)


def grads_of(fn, inputs, cots):
    leaves = [x.detach().clone().requires_grad_(True) for x in inputs]
    outs = fn(*leaves)
    outs_t = outs if isinstance(outs, tuple) else (outs,)
    cots = cots if isinstance(cots, (tuple, list)) else (cots,)
    loss = sum((o.float() * c.float()).sum() for o, c in zip(outs_t, cots))
    return outs, torch.autograd.grad(loss, leaves)


FUSED = {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}
QK = {1: nb.na1d_qk, 2: nb.na2d_qk, 3: nb.na3d_qk}
AV = {1: nb.na1d_av, 2: nb.na2d_av, 3: nb.na3d_av}
VARLEN = {1: nb.na1d_varlen, 2: nb.na2d_varlen, 3: nb.na3d_varlen}


# ---------------------------------------------------------------------------
# 1. every golden case: CUDA result == the reference's own result
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("idx", range(len(CASES)))
def test_golden_case_on_cuda(idx, golden_cases):
    cases, ref = golden_cases
    case = cases[idx]
    x = {k: torch.from_numpy(v).to(DEV) for k, v in make_inputs(idx, case).items()}
    rank = len(case["shape"]) - 3
    ks, st = tup(case["kernel_size"], rank), tup(case["stride"], rank)
    dl, ca = tup(case["dilation"], rank), tup(case["is_causal"], rank)
    kind = case["kind"]
    g = lambda name: ref[f"c{idx}_{name}"]
    if kind == "fused":
        fn = lambda q, k, v: FUSED[rank](q, k, v, kernel_size=ks, stride=st, dilation=dl, is_causal=ca)
        out, gr = grads_of(fn, [x["q"], x["k"], x["v"]], x["cot"])
        close32(out, g("out"), "out")
        for name, t in zip(("dq", "dk", "dv"), gr):
            close32(t, g(name), name)
    elif kind == "qk":
        fn = lambda q, k: QK[rank](q, k, ks, dl, stride=st, is_causal=ca)
        out = fn(x["q"], x["k"])
        close32(out, g("out"), "logits")
        # cotangent on -inf slots is ignored by the backward (masked slots get zero gradient)
        _, gr = grads_of(lambda q, k: torch.nan_to_num(fn(q, k), neginf=0.0), [x["q"], x["k"]], x["cot"])
        close32(gr[0], g("dq"), "dq")
        close32(gr[1], g("dk"), "dk")
    elif kind == "av":
        fn = lambda a, v: AV[rank](a, v, ks, dl, stride=st, is_causal=ca)
        out, gr = grads_of(fn, [x["attn"], x["v"]], x["cot"])
        close32(out, g("out"), "out")
        close32(gr[0], g("dattn"), "dattn")
        close32(gr[1], g("dv"), "dv")
    elif kind == "lse_extra":
        names = ["q", "k", "v"] + (["ak", "av"] if "ak" in x else [])

        def fn(*a):
            kw = dict(additional_keys=a[3], additional_values=a[4]) if len(a) == 5 else {}
            return FUSED[rank](a[0], a[1], a[2], kernel_size=ks, stride=st, dilation=dl, is_causal=ca,
                               return_lse=True, **kw)
        (out, lse), gr = grads_of(fn, [x[n] for n in names], (x["cot"], x["cot_lse"]))
        close32(out, g("out"), "out")
        close32(lse, g("lse"), "lse")
        for n, t in zip(names, gr):
            close32(t, g("d" + n), "d" + n)
    elif kind == "varlen":
        sizes = torch.tensor(case["sizes"], dtype=torch.int32, device=DEV)
        if rank == 1:
            sizes = sizes.reshape(-1)
        fn = lambda q, k, v: VARLEN[rank](q, k, v, sizes, ks, dl)
        out, gr = grads_of(fn, [x["q"], x["k"], x["v"]], x["cot"])
        close32(out, g("out"), "out")
        for name, t in zip(("dq", "dk", "dv"), gr):
            close32(t, g(name), name)
    elif kind == "merge":
        n = case["n_parts"]
        out, lse = nb.merge_attentions([x[f"o{j}"] for j in range(n)], [x[f"l{j}"] for j in range(n)])
        close32(out, g("out"), "out")
        close32(lse, g("lse"), "lse")
    elif kind == "qk_rpb":
        f = allin1.na1d_qk_rpb if rank == 1 else allin1.na2d_qk_rpb
        close32(f(x["q"], x["k"], x.get("rpb"), case["kernel_size"], case["dilation"], scale=0.288), g("out"), "logits")
    elif kind == "av_fused":
        f = allin1.na1d_av_fused if rank == 1 else allin1.na2d_av_fused
        close32(f(x["attn"], x["v"], case["kernel_size"], case["dilation"]), g("out"), "out")


# ---------------------------------------------------------------------------
# 2. neighbour index and mask, bit-exact, read through the split-QK logits
# ---------------------------------------------------------------------------
def _index_logits(extent, ks, st, dl, ca):
    """q = 1, k = linear position, D = 1, scale = 1 -> logits are the key indices."""
    n = int(np.prod(extent))
    q = torch.ones((1,) + tuple(extent) + (1, 1), device=DEV)
    k = torch.arange(n, dtype=torch.float32, device=DEV).reshape((1,) + tuple(extent) + (1, 1))
    rank = len(extent)
    return QK[rank](q, k, ks, dl, stride=st, is_causal=ca, scale=1.0)[0, ..., 0, :].cpu().numpy()


def test_index_and_mask_bit_exact_1d_exhaustive():
    for K, d, s, causal in itertools.product([1, 2, 3, 4, 5, 7], [1, 2, 3, 4], [1, 2, 3], [False, True]):
        if s > K:
            continue
        for L in range(K * d, K * d + 11):
            got = _index_logits((L,), (K,), (s,), (d,), (causal,))
            lin, ok, _ = oracle.neighbor_tables((L,), (K,), (s,), (d,), (causal,))
            want = np.where(ok, lin.astype(np.float32), -np.inf)
            assert np.array_equal(got, want), (L, K, d, s, causal)


@pytest.mark.parametrize("extent,ks,st,dl,ca", [
    ((9, 11), (3, 5), (1, 1), (2, 1), (False, False)),
    ((12, 10), (5, 3), (2, 1), (1, 3), (True, False)),
    ((8, 8), (4, 6), (1, 2), (2, 1), (False, True)),
    ((56, 56), (7, 7), (1, 1), (4, 4), (False, False)),
    ((5, 7, 8), (3, 3, 5), (1, 1, 1), (1, 2, 1), (True, False, False)),
    ((6, 9, 7), (3, 3, 3), (1, 2, 1), (2, 3, 1), (False, False, True)),
    ((4, 16, 16), (3, 7, 7), (1, 1, 1), (1, 2, 2), (True, False, False)),
])
def test_index_and_mask_bit_exact_nd(extent, ks, st, dl, ca):
    got = _index_logits(extent, ks, st, dl, ca)
    lin, ok, _ = oracle.neighbor_tables(extent, ks, st, dl, ca)
    want = np.where(ok, lin.astype(np.float32), -np.inf)
    assert np.array_equal(got, want)


# ---------------------------------------------------------------------------
# 3. low precision against the float32 oracle
# ---------------------------------------------------------------------------
def _rand(shape, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,ks,st,dl,ca,hkv", [
    ((2, 40, 4, 32), (7,), (1,), (2,), (False,), 4),
    ((1, 33, 4, 64), (5,), (2,), (1,), (True,), 2),
    ((2, 18, 20, 4, 32), (7, 7), (1, 1), (1, 2), (False, False), 4),
    ((1, 16, 16, 4, 64), (5, 3), (2, 1), (1, 1), (False, True), 1),
    ((1, 4, 14, 15, 2, 64), (3, 7, 7), (1, 1, 1), (1, 2, 2), (True, False, False), 2),
])
def test_low_precision_fused_forward_backward(dtype, shape, ks, st, dl, ca, hkv):
    rank = len(shape) - 3
    kv_shape = shape[:-2] + (hkv, shape[-1])
    q, k, v = _rand(shape, 1, dtype), _rand(kv_shape, 2, dtype), _rand(kv_shape, 3, dtype)
    outs = tuple(-(-shape[1 + a] // st[a]) for a in range(rank))
    cot = _rand((shape[0],) + outs + shape[-2:], 4, dtype)
    cot_l = _rand((shape[0],) + outs + (shape[-2],), 5)
    fn_ref = lambda q_, k_, v_: oracle.na(q_, k_, v_, ks, st, dl, ca, return_lse=True)
    (o_ref, l_ref), g_ref = oracle.grads(fn_ref, [q.float(), k.float(), v.float()], (cot.float(), cot_l))
    fn = lambda q_, k_, v_: FUSED[rank](q_, k_, v_, kernel_size=ks, stride=st, dilation=dl, is_causal=ca, return_lse=True)
    (o, l), g = grads_of(fn, [q.to(DEV), k.to(DEV), v.to(DEV)], (cot.to(DEV), cot_l.to(DEV)))
    assert o.dtype == dtype and l.dtype == torch.float32
    close_lowp(o, o_ref, "out")
    close_lowp(l, l_ref, "lse")
    for name, a, b in zip(("dq", "dk", "dv"), g, g_ref):
        assert a.dtype == dtype
        close_lowp(a, b, name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_low_precision_split_ops(dtype):
    shape, ks, st, dl, ca = (1, 12, 14, 2, 32), (3, 5), (1, 2), (2, 1), (False, True)
    q, k = _rand(shape, 11, dtype), _rand(shape, 12, dtype)
    want = oracle.na_qk(q.float(), k.float(), ks, st, dl, ca)
    got = nb.na2d_qk(q.to(DEV), k.to(DEV), ks, dl, stride=st, is_causal=ca)
    assert got.dtype == dtype
    close_lowp(got, want, "logits")
    attn = torch.softmax(want, -1)
    got_o = nb.na2d_av(attn.to(dtype).to(DEV), k.to(DEV), ks, dl, stride=st, is_causal=ca)
    close_lowp(got_o, oracle.na_av(attn.to(dtype).float(), k.float(), ks, st, dl, ca), "av")


# ---------------------------------------------------------------------------
# 4. the named configurations (reduced where the oracle would not fit in time)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dil", [1, 4])
def test_config_na2d_bf16_nat_stage(dil):
    """na2d bf16, 56x56, 4 heads, D=32, K=7x7, dilation 1 and 4 (batch 2 of the 32)."""
    shape = (2, 56, 56, 4, 32)
    q, k, v, cot = (_rand(shape, 1234 + i, torch.bfloat16) for i in range(4))
    fn_ref = lambda a, b, c: oracle.na(a, b, c, (7, 7), 1, dil, False)
    o_ref, g_ref = oracle.grads(fn_ref, [q.float(), k.float(), v.float()], cot.float())
    fn = lambda a, b, c: nb.na2d(a, b, c, kernel_size=7, dilation=dil)
    o, g = grads_of(fn, [q.to(DEV), k.to(DEV), v.to(DEV)], cot.to(DEV))
    close_lowp(o, o_ref, "out")
    for name, a, b in zip(("dq", "dk", "dv"), g, g_ref):
        close_lowp(a, b, name)


def test_config_allin1_split_1d_fp32():
    """na1d_qk_rpb -> softmax -> na1d_av_fused, B=8, L=4096, H=4, D=12, K=5, dilation 2, scale 0.288."""
    shape = (8, 4096, 4, 12)
    q, k, v = _rand(shape, 21), _rand(shape, 22), _rand(shape, 23)
    rpb = _rand((4, 9), 24) * 0.02
    want_l = oracle.qk_rpb(q, k, rpb, 5, 2, 0.288)
    want_o = oracle.av_fused(torch.softmax(want_l, -1), v, 5, 2)
    logits = allin1.na1d_qk_rpb(q.to(DEV), k.to(DEV), rpb.to(DEV), 5, 2, scale=0.288)
    out = allin1.na1d_av_fused(torch.softmax(logits, -1), v.to(DEV), 5, 2)
    close32(logits, want_l, "logits")
    close32(out, want_o, "out")


def test_allin1_fused_forward_matches_split_and_oracle():
    """QK + RPB -> softmax -> AV in one launch equals the split composition and the oracle (float32 1e-4; bf16 2e-2)."""
    shape = (8, 4096, 4, 12)
    q, k, v = _rand(shape, 21), _rand(shape, 22), _rand(shape, 23)
    rpb = _rand((4, 9), 24) * 0.02
    want = oracle.av_fused(torch.softmax(oracle.qk_rpb(q, k, rpb, 5, 2, 0.288), -1), v, 5, 2)
    before = _lib.launch_count()
    got = allin1.na1d_qkv_fused(q.to(DEV), k.to(DEV), v.to(DEV), rpb.to(DEV), 5, 2, scale=0.288)
    assert _lib.launch_count() - before == 1
    close32(got, want, "fused 1d")
    # 2D, no bias, and with bias
    shape = (2, 9, 12, 2, 12)
    q, k, v = _rand(shape, 41), _rand(shape, 42), _rand(shape, 43)
    rpb = _rand((2, 5, 5), 44) * 0.02
    for r in (None, rpb):
        want = oracle.av_fused(torch.softmax(oracle.qk_rpb(q, k, r, 3, 2, 0.288), -1), v, 3, 2)
        got = allin1.na2d_qkv_fused(q.to(DEV), k.to(DEV), v.to(DEV), None if r is None else r.to(DEV), 3, 2, scale=0.288)
        close32(got, want, "fused 2d")
    # bf16, head dim 32
    shape = (1, 14, 10, 2, 32)
    q, k, v = (_rand(shape, 50 + i, torch.bfloat16) for i in range(3))
    want = oracle.av_fused(torch.softmax(oracle.qk_rpb(q.float(), k.float(), None, 5, 1, 32 ** -0.5), -1), v.float(), 5, 1)
    got = allin1.na2d_qkv_fused(q.to(DEV), k.to(DEV), v.to(DEV), None, 5, 1, scale=32 ** -0.5)
    close_lowp(got, want, "fused 2d bf16")
    with pytest.raises(ValueError, match="head_dim"):
        allin1.na1d_qkv_fused(torch.randn(1, 16, 2, 20, device=DEV), torch.randn(1, 16, 2, 20, device=DEV),
                              torch.randn(1, 16, 2, 20, device=DEV), None, 3)


def test_allin1_gradients_match_autograd_of_oracle():
    shape = (2, 30, 2, 12)
    q, k, v = _rand(shape, 31), _rand(shape, 32), _rand(shape, 33)
    rpb = _rand((2, 9), 34) * 0.02
    cot = _rand(shape, 35)
    ref = lambda q_, k_, r_, v_: oracle.av_fused(torch.softmax(oracle.qk_rpb(q_, k_, r_, 5, 2, 0.288), -1), v_, 5, 2)
    o_ref, g_ref = oracle.grads(ref, [q, k, rpb, v], cot)
    fn = lambda q_, k_, r_, v_: allin1.na1d_av_fused(torch.softmax(allin1.na1d_qk_rpb(q_, k_, r_, 5, 2, scale=0.288), -1), v_, 5, 2)
    o, g = grads_of(fn, [t.to(DEV) for t in (q, k, rpb, v)], cot.to(DEV))
    close32(o, o_ref, "out")
    for name, a, b in zip(("dq", "dk", "drpb", "dv"), g, g_ref):
        close32(a, b, name)
    # 2D
    shape = (1, 9, 12, 2, 12)
    q, k, v = _rand(shape, 41), _rand(shape, 42), _rand(shape, 43)
    rpb = _rand((2, 5, 5), 44) * 0.02
    cot = _rand(shape, 45)
    ref = lambda q_, k_, r_, v_: oracle.av_fused(torch.softmax(oracle.qk_rpb(q_, k_, r_, 3, 2, 0.288), -1), v_, 3, 2)
    o_ref, g_ref = oracle.grads(ref, [q, k, rpb, v], cot)
    fn = lambda q_, k_, r_, v_: allin1.na2d_av_fused(torch.softmax(allin1.na2d_qk_rpb(q_, k_, r_, 3, 2, scale=0.288), -1), v_, 3, 2)
    o, g = grads_of(fn, [t.to(DEV) for t in (q, k, rpb, v)], cot.to(DEV))
    close32(o, o_ref, "out")
    for name, a, b in zip(("dq", "dk", "drpb", "dv"), g, g_ref):
        close32(a, b, name)


def test_config_na3d_bf16_video_reduced():
    """na3d bf16, K=(3,7,7), causal along T, dilation (1,2,2), D=64 (T=6, 16x18, 2 heads of the full shape)."""
    shape = (1, 6, 16, 18, 2, 64)
    q, k, v, cot = (_rand(shape, 50 + i, torch.bfloat16) for i in range(4))
    ks, dl, ca = (3, 7, 7), (1, 2, 2), (True, False, False)
    o_ref, g_ref = oracle.grads(lambda a, b, c: oracle.na(a, b, c, ks, 1, dl, ca), [q.float(), k.float(), v.float()], cot.float())
    o, g = grads_of(lambda a, b, c: nb.na3d(a, b, c, kernel_size=ks, dilation=dl, is_causal=ca),
                    [q.to(DEV), k.to(DEV), v.to(DEV)], cot.to(DEV))
    close_lowp(o, o_ref, "out")
    for name, a, b in zip(("dq", "dk", "dv"), g, g_ref):
        close_lowp(a, b, name)


def test_config_na2d_varlen_gqa_extra_tokens_reduced():
    """na2d bf16 varlen + GQA + extra tokens + LSE, K=13x13, dilation 2, D=128
    (B=3 padded to 40x40, sizes from {26, 32, 40}, 8 query / 2 KV heads -- four query heads share a tile --
    and 24 extra tokens)."""
    B, M, Hq, Hkv, D, NE = 3, 40, 8, 2, 128, 24
    sizes = [[40, 26], [26, 32], [32, 40]]
    q = _rand((B, M, M, Hq, D), 60, torch.bfloat16)
    k, v = _rand((B, M, M, Hkv, D), 61, torch.bfloat16), _rand((B, M, M, Hkv, D), 62, torch.bfloat16)
    ak, av = _rand((B, NE, Hkv, D), 63, torch.bfloat16), _rand((B, NE, Hkv, D), 64, torch.bfloat16)
    cot, cot_l = _rand((B, M, M, Hq, D), 65, torch.bfloat16), _rand((B, M, M, Hq), 66)
    # padded cotangents never reach the gradients
    ref = lambda q_, k_, v_, ak_, av_: oracle.na_varlen(q_, k_, v_, sizes, 13, 2, return_lse=True,
                                                        additional_keys=ak_, additional_values=av_)
    (o_ref, l_ref), g_ref = oracle.grads(ref, [t.float() for t in (q, k, v, ak, av)], (cot.float(), cot_l))
    st = torch.tensor(sizes, dtype=torch.int32, device=DEV)
    fn = lambda q_, k_, v_, ak_, av_: nb.na2d_varlen(q_, k_, v_, st, 13, 2, return_lse=True,
                                                     additional_keys=ak_, additional_values=av_, host_sizes=sizes)
    (o, l), g = grads_of(fn, [t.to(DEV) for t in (q, k, v, ak, av)], (cot.to(DEV), cot_l.to(DEV)))
    close_lowp(o, o_ref, "out")
    close_lowp(l, l_ref, "lse")
    for name, a, b in zip(("dq", "dk", "dv", "dak", "dav"), g, g_ref):
        close_lowp(a, b, name)
    # padding is exactly zero in outputs and gradients
    for b, (h, w) in enumerate(sizes):
        for t in (o,) + tuple(g[:3]):
            assert t[b, h:].abs().sum() == 0 and t[b, :, w:].abs().sum() == 0


# ---------------------------------------------------------------------------
# 5. size-independent properties at the full benchmark size
# ---------------------------------------------------------------------------
def test_full_size_properties_na2d_bf16():
    shape = (32, 56, 56, 4, 32)
    g_ = torch.Generator(device=DEV).manual_seed(7)
    q, k, v, cot = (torch.randn(shape, generator=g_, device=DEV).to(torch.bfloat16) for _ in range(4))
    for dil in (1, 4):
        fn = lambda a, b, c: nb.na2d(a, b, c, kernel_size=7, dilation=dil, return_lse=True)
        with torch.no_grad():
            o, lse = fn(q, k, v)
        # rows of the softmax sum to one: attention over constant values returns the constant
        ones = torch.ones_like(v)
        assert (nb.na2d(q, k, ones, kernel_size=7, dilation=dil).float() - 1).abs().max() < 1e-2
        # fused == split composition, and lse == logsumexp of the split logits
        logits = nb.na2d_qk(q, k, 7, dil).float()
        o_split = nb.na2d_av(torch.softmax(logits, -1).to(torch.bfloat16), v, 7, dil)
        # both sides round probabilities and outputs to bf16: 2e-2 of the largest magnitude, as everywhere
        assert (o.float() - o_split.float()).abs().max() / o.float().abs().max() < 2e-2
        assert (lse - torch.logsumexp(logits, -1)).abs().max() < 3e-2
        # gradient identities: sum_keys dV = sum_queries dO ; sum q.dq = sum k.dk (rows of dS sum to zero)
        _, (dq, dk, dv) = grads_of(lambda a, b, c: nb.na2d(a, b, c, kernel_size=7, dilation=dil), [q, k, v], cot)
        lhs, rhs = dv.float().sum((1, 2)), cot.float().sum((1, 2))
        assert (lhs - rhs).abs().max() / rhs.abs().max() < 2e-2
        a = (q.float() * dq.float()).sum((1, 2, 4))
        b = (k.float() * dk.float()).sum((1, 2, 4))
        assert (a - b).abs().max() / a.abs().max().clamp_min(1.0) < 5e-2
        # same inputs, same bits
        o2 = nb.na2d(q, k, v, kernel_size=7, dilation=dil)
        assert torch.equal(o, o2)


def test_full_size_properties_na3d_video_bf16():
    """The video volume at full size (bf16 B=2 T=32 96x96 16 heads D=64, kernel (3,7,7), causal along T, dilation
    (1,2,2)): softmax rows sum to one, the leading planes equal a call on those planes alone (causal axis), fused ==
    split composition on a slab, sum_keys dV == sum_queries dO, same inputs give the same bits, no wait ran out."""
    shape, ks, dl, ca = (2, 32, 96, 96, 16, 64), (3, 7, 7), (1, 2, 2), (True, False, False)
    g_ = torch.Generator(device=DEV).manual_seed(11)
    q, k, v, cot = (torch.randn(shape, generator=g_, device=DEV).to(torch.bfloat16) for _ in range(4))
    fn = lambda a, b, c: nb.na3d(a, b, c, kernel_size=ks, dilation=dl, is_causal=ca, return_lse=True)
    with torch.no_grad():
        o, lse = fn(q, k, v)
        assert _lib.last_path() == "tcgen05"
        assert (nb.na3d(q, k, torch.ones_like(v), kernel_size=ks, dilation=dl, is_causal=ca).float() - 1).abs().max() < 1e-2
        # causal along T: planes [0, 6) depend on nothing later
        o6, lse6 = fn(q[:, :6].contiguous(), k[:, :6].contiguous(), v[:, :6].contiguous())
        assert (o[:, :6].float() - o6.float()).abs().max() / o6.float().abs().max() < 1e-2
        assert (lse[:, :6] - lse6).abs().max() < 1e-2
        # fused == split on a slab of four planes and four heads
        qs, ks_, vs = (t[:1, :4, :, :, 4:8].contiguous() for t in (q, k, v))
        logits = nb.na3d_qk(qs, ks_, ks, dl, is_causal=ca).float()
        o_split = nb.na3d_av(torch.softmax(logits, -1).to(torch.bfloat16), vs, ks, dl, is_causal=ca)
        assert (o[:1, :4, :, :, 4:8].float() - o_split.float()).abs().max() / o_split.float().abs().max() < 2e-2
        assert (lse[:1, :4, :, :, 4:8] - torch.logsumexp(logits, -1)).abs().max() < 3e-2
    _, (dq, dk, dv) = grads_of(lambda a, b, c: nb.na3d(a, b, c, kernel_size=ks, dilation=dl, is_causal=ca), [q, k, v], cot)
    lhs, rhs = dv.float().sum((1, 2, 3)), cot.float().sum((1, 2, 3))
    assert (lhs - rhs).abs().max() / rhs.abs().max() < 2e-2
    a = (q.float() * dq.float()).sum((1, 2, 3, 5))
    b = (k.float() * dk.float()).sum((1, 2, 3, 5))
    assert (a - b).abs().max() / a.abs().max().clamp_min(1.0) < 5e-2
    with torch.no_grad():
        assert torch.equal(o, fn(q, k, v)[0])
    assert _lib.kernel_status() == 0


def test_video_geometry_slice_against_the_oracle():
    """Three planes of the video geometry at its full 96x96 extent and 16 heads on the GPU; two of the heads against
    the CPU oracle (out, lse and all gradients)."""
    shape, ks, dl, ca = (1, 3, 96, 96, 16, 64), (3, 7, 7), (1, 2, 2), (True, False, False)
    q, k, v, cot = (_rand(shape, 300 + i, torch.bfloat16) for i in range(4))
    cot_l = _rand(shape[:-1], 305)
    hs = slice(5, 7)
    ref = lambda a, b, c: oracle.na(a, b, c, ks, 1, dl, ca, return_lse=True)
    (o_ref, l_ref), g_ref = oracle.grads(ref, [t[..., hs, :].float() for t in (q, k, v)],
                                         (cot[..., hs, :].float(), cot_l[..., hs]))
    fn = lambda a, b, c: nb.na3d(a, b, c, kernel_size=ks, dilation=dl, is_causal=ca, return_lse=True)
    (o, l), g = grads_of(fn, [t.to(DEV) for t in (q, k, v)], (cot.to(DEV), cot_l.to(DEV)))
    assert _lib.last_path() == "tcgen05" and _lib.kernel_status() == 0
    close_lowp(o[..., hs, :], o_ref, "out")
    close_lowp(l[..., hs], l_ref, "lse")
    for name, a, b in zip(("dq", "dk", "dv"), g, g_ref):
        close_lowp(a[..., hs, :], b, name)


def test_full_size_properties_varlen_gqa_extra_tokens_bf16():
    """The variable-size GQA batch at full size (bf16 B=16 padded to 128x128, sizes from {64,...,128}, 16 query / 4 KV
    heads, D=128, kernel 13x13, dilation 2, 64 extra tokens, LSE): one launch forward and four backward, rows sum to
    one, padding is zero, a sample equals the dense call on its own tensors, the value gradients sum to the output
    cotangent, same inputs give the same bits."""
    B, M, Hq, Hkv, D, NX = 16, 128, 16, 4, 128, 64
    gen = torch.Generator().manual_seed(1236)
    sizes = (torch.randint(0, 9, (B, 2), generator=gen) * 8 + 64).tolist()
    g_ = torch.Generator(device=DEV).manual_seed(12)
    rnd = lambda *s_: torch.randn(s_, generator=g_, device=DEV).to(torch.bfloat16)
    q, k, v = rnd(B, M, M, Hq, D), rnd(B, M, M, Hkv, D), rnd(B, M, M, Hkv, D)
    ak, av, cot = rnd(B, NX, Hkv, D), rnd(B, NX, Hkv, D), rnd(B, M, M, Hq, D)
    st = torch.tensor(sizes, dtype=torch.int32, device=DEV)
    mask = torch.zeros(B, M, M, dtype=torch.bool, device=DEV)
    for b, (h, w) in enumerate(sizes):
        mask[b, :h, :w] = True
    call = lambda q_, k_, v_, ak_, av_: nb.na2d_varlen(q_, k_, v_, st, 13, 2, return_lse=True, additional_keys=ak_,
                                                       additional_values=av_, host_sizes=sizes)
    leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v, ak, av)]
    n0 = _lib.launch_count()
    o, lse = call(*leaves)
    assert _lib.last_path() == "tcgen05" and _lib.launch_count() - n0 == 1
    n1 = _lib.launch_count()
    dq, dk, dv, dak, dav = torch.autograd.grad(o, leaves, cot)
    assert _lib.launch_count() - n1 == 4
    assert _lib.kernel_status() == 0
    with torch.no_grad():
        ones = call(q, k, torch.ones_like(v), ak, torch.ones_like(av))[0].float()
        assert (ones[mask] - 1).abs().max() < 1e-2
        for t in (o, lse, dq, dk, dv):
            assert float(t[~mask].abs().sum()) == 0.0
        # sample 3 alone, as a dense call on its own tensors
        b = 3
        h, w = sizes[b]
        ob, lb = nb.na2d(q[b:b + 1, :h, :w].contiguous(), k[b:b + 1, :h, :w].contiguous(), v[b:b + 1, :h, :w].contiguous(),
                         kernel_size=13, dilation=2, return_lse=True, additional_keys=ak[b:b + 1], additional_values=av[b:b + 1])
        assert (o[b, :h, :w].float() - ob[0].float()).abs().max() / ob.float().abs().max() < 1e-2
        assert (lse[b, :h, :w] - lb[0]).abs().max() < 1e-2
        # every query's weights sum to one, so the value gradients (window keys + extra tokens) carry all of dO
        rhs = (cot.float() * mask[..., None, None]).reshape(B, M * M, Hkv, Hq // Hkv, D).sum((1, 3))
        lhs = dv.float().sum((1, 2)) + dav.float().sum(1)
        assert (lhs - rhs).abs().max() / rhs.abs().max() < 2e-2
        assert torch.equal(o, call(q, k, v, ak, av)[0])


def test_known_answers():
    # causal first position attends to itself only (tests/test_functional.py:253-262 of the reference)
    q = torch.randn(1, 8, 1, 4, device=DEV)
    v = torch.arange(8, dtype=torch.float32, device=DEV).reshape(1, 8, 1, 1).expand(1, 8, 1, 4).contiguous()
    out = nb.na1d(q, q, v, kernel_size=3, is_causal=True)
    assert float(out[0, 0, 0, 0]) == 0.0
    # kernel covering the extent == global attention (tests/test_functional.py:122-139)
    q, k, v = (torch.randn(2, 9, 2, 8, device=DEV) for _ in range(3))
    want = torch.softmax(torch.einsum("blhd,bmhd->bhlm", q, k) * 8 ** -0.5, -1)
    want = torch.einsum("bhlm,bmhd->blhd", want, v)
    close32(nb.na1d(q, k, v, kernel_size=9), want, "global")
    # GQA == explicit repeat (tests/test_new_features.py:350-368)
    q = torch.randn(1, 10, 12, 4, 8, device=DEV)
    k, v = torch.randn(1, 10, 12, 2, 8, device=DEV), torch.randn(1, 10, 12, 2, 8, device=DEV)
    a = nb.na2d(q, k, v, kernel_size=3)
    b = nb.na2d(q, k.repeat_interleave(2, dim=-2), v.repeat_interleave(2, dim=-2), kernel_size=3)
    close32(a, b, "gqa")
    # merging two windows over split key sets == attention over the union (tests/test_new_features.py:235-255)
    q = torch.randn(1, 6, 2, 8, device=DEV)
    ka, va, kb, vb = (torch.randn(1, 6, 2, 8, device=DEV) for _ in range(4))
    oa, la = nb.na1d(q, ka, va, kernel_size=6, return_lse=True)
    ob, lb = nb.na1d(q, kb, vb, kernel_size=6, return_lse=True)
    om, lm = nb.merge_attentions([oa, ob], [la, lb])
    kk, vv = torch.cat([ka, kb], 1), torch.cat([va, vb], 1)
    s = torch.einsum("blhd,bmhd->bhlm", q, kk) * 8 ** -0.5
    close32(om, torch.einsum("bhlm,bmhd->blhd", torch.softmax(s, -1), vv), "merged out")
    close32(lm, torch.logsumexp(s, -1).permute(0, 2, 1), "merged lse")


def test_merge_gradients():
    o = [_rand((2, 5, 3, 8), 70 + i) for i in range(3)]
    l = [_rand((2, 5, 3), 80 + i) * 2 for i in range(3)]
    cot, cot_l = _rand((2, 5, 3, 8), 90), _rand((2, 5, 3), 91)
    ref = lambda *a: oracle.merge_attentions(list(a[:3]), list(a[3:]))
    _, g_ref = oracle.grads(ref, o + l, (cot, cot_l))
    fn = lambda *a: nb.merge_attentions(list(a[:3]), list(a[3:]))
    _, g = grads_of(fn, [t.to(DEV) for t in o + l], (cot.to(DEV), cot_l.to(DEV)))
    for i, (a, b) in enumerate(zip(g, g_ref)):
        close32(a, b, f"grad{i}")


# ---------------------------------------------------------------------------
# 6. the CUDA library is what runs; nothing falls back
# ---------------------------------------------------------------------------
def test_library_launches_and_reports_path():
    q = torch.randn(1, 16, 2, 12, device=DEV)
    before = _lib.launch_count()
    nb.na1d(q, q, q, kernel_size=3)
    assert _lib.launch_count() > before
    assert _lib.last_path() in ("simt", "tcgen05")
    nb.set_fused_path("tcgen05")
    try:
        with pytest.raises(ValueError, match="tcgen05"):
            nb.na1d(q, q, q, kernel_size=3)          # float32, D=12: no tensor-core kernel, and no fallback
    finally:
        nb.set_fused_path("auto")


# ---------------------------------------------------------------------------
# 7. slab of a larger volume (leading-axis shard with halo) == the unsharded result
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("causal_t", [True, False])
def test_leading_axis_slabs_match_unsharded(causal_t):
    from natten_mlx_b200.sharding import slab_plan, fused_slab_forward_backward
    shape = (1, 12, 9, 10, 2, 16)
    ks, dl, ca = (3, 3, 5), (2, 1, 1), (causal_t, False, False)
    q, k, v, cot = (_rand(shape, 100 + i).to(DEV) for i in range(4))
    o_ref, g_ref = grads_of(lambda a, b, c: nb.na3d(a, b, c, kernel_size=ks, dilation=dl, is_causal=ca), [q, k, v], cot)
    T, world = shape[1], 2
    dk_full, dv_full = torch.zeros_like(k), torch.zeros_like(v)
    for rank_ in range(world):
        plan = slab_plan(T, world, rank_, ks[0], dl[0], ca[0])
        qs = q[:, plan.q_lo:plan.q_hi]
        ks_, vs_ = k[:, plan.kv_lo:plan.kv_hi], v[:, plan.kv_lo:plan.kv_hi]
        o, lse, dq, dk_, dv_ = fused_slab_forward_backward(qs, ks_, vs_, cot[:, plan.q_lo:plan.q_hi], plan, shape[1:4],
                                                           ks, dl, ca, None)
        close32(o, o_ref[:, plan.q_lo:plan.q_hi], "slab out")
        close32(dq, g_ref[0][:, plan.q_lo:plan.q_hi], "slab dq")
        dk_full[:, plan.kv_lo:plan.kv_hi] += dk_
        dv_full[:, plan.kv_lo:plan.kv_hi] += dv_
    close32(dk_full, g_ref[1], "dk (halo partials added)")
    close32(dv_full, g_ref[2], "dv (halo partials added)")
