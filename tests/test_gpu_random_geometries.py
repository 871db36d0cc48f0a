"""Seeded random geometries through both kernel families: the tensor-core kernels (bf16) against the
CUDA-core kernels run in float32 on the same values, forward and backward, with the features mixed at
random (rank, head dim, GQA, kernel, dilation, causal axes, stride, extra tokens, per-sample sizes).
The float32 CUDA-core path is itself checked against the CPU oracle elsewhere; here it stands in for
it so that a few hundred geometries fit into seconds.  Tolerance: 2e-2 of the largest reference
magnitude and 5e-2 per element, as everywhere for bf16."""

from __future__ import annotations

import random

import pytest
import torch

from conftest import assert_lowp

from natten_mlx_b200 import _lib
from natten_mlx_b200._core import cuda as backend

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _geometry(rng):
    rank = rng.choice([1, 2, 2, 2, 3])
    D = rng.choice([32, 32, 64, 128])
    hkv = rng.choice([1, 2])
    rep = rng.choice([1, 1, 2, 4])
    ks, dl, ca, ext = [], [], [], []
    for a in range(rank):
        k = rng.choice([3, 4, 5, 7] if rank > 1 else [3, 5, 7, 13, 31])
        d = rng.choice([1, 1, 2, 3])
        lo = k * d
        ext.append(rng.randint(lo, lo + (24 if rank < 3 else 8)))
        ks.append(k)
        dl.append(d)
        ca.append(rng.random() < 0.25)
    st = [1] * rank
    mode = rng.choice(["plain", "plain", "stride", "extra", "varlen", "varlen_extra"])
    if mode == "stride":
        for a in range(rank):
            if dl[a] == 1 and rng.random() < 0.7:
                st[a] = rng.randint(1, min(ks[a], 3))
    if mode.startswith("varlen"):
        ca = [False] * rank
    B = rng.choice([1, 2, 3])
    return dict(rank=rank, D=D, hkv=hkv, hq=hkv * rep, ks=tuple(ks), dl=tuple(dl), ca=tuple(ca), st=tuple(st),
                ext=tuple(ext), B=B, mode=mode, n_extra=rng.choice([3, 17, 40]) if "extra" in mode else 0)


@pytest.mark.parametrize("seed", range(6))
def test_tensor_core_kernels_agree_with_the_float32_kernels_on_random_geometries(seed):
    rng = random.Random(4100 + seed)
    ran = 0
    for case in range(40):
        g = _geometry(rng)
        gen = torch.Generator().manual_seed(seed * 1000 + case)
        mk = lambda shape: torch.randn(shape, generator=gen).to(torch.bfloat16).to(DEV)
        q = mk((g["B"],) + g["ext"] + (g["hq"], g["D"]))
        k, v = (mk((g["B"],) + g["ext"] + (g["hkv"], g["D"])) for _ in range(2))
        ke = ve = None
        if g["n_extra"]:
            ke, ve = (mk((g["B"], g["n_extra"], g["hkv"], g["D"])) for _ in range(2))
        sizes = host = None
        if g["mode"].startswith("varlen"):
            host = [tuple(rng.randint(g["ks"][a] * g["dl"][a], g["ext"][a]) for a in range(g["rank"])) for _ in range(g["B"])]
            sizes = torch.tensor(host, dtype=torch.int32, device=DEV)
        kw = dict(k_extra=ke, v_extra=ve, sizes=sizes, host_sizes=host)
        args = (g["ks"], g["st"], g["dl"], g["ca"], None)
        try:
            out, lse = backend.fused_forward(q, k, v, *args, path="tcgen05", **kw)
        except ValueError:
            continue                      # a geometry the tensor-core planner does not take
        assert _lib.last_path() == "tcgen05"
        cot = mk(tuple(out.shape))
        dlse = torch.randn(lse.shape, generator=gen).to(DEV) if rng.random() < 0.5 else None
        grads = backend.fused_backward(q, k, v, out, lse, cot, dlse, *args, path="tcgen05", **kw)
        f = lambda t: None if t is None else t.float()
        kw32 = dict(k_extra=f(ke), v_extra=f(ve), sizes=sizes, host_sizes=host)
        out32, lse32 = backend.fused_forward(q.float(), k.float(), v.float(), *args, path="simt", **kw32)
        grads32 = backend.fused_backward(q.float(), k.float(), v.float(), out32, lse32, cot.float(), dlse, *args,
                                         path="simt", **kw32)
        assert _lib.last_path() == "simt"
        tag = f"seed {seed} case {case} {g}"
        assert_lowp(out, out32, "out " + tag)
        assert_lowp(lse, lse32, "lse " + tag)
        for name, a, b in zip(("dq", "dk", "dv", "dk_extra", "dv_extra"), grads, grads32):
            if a is not None:
                assert_lowp(a, b, name + " " + tag)
        ran += 1
    assert _lib.kernel_status() == 0
    assert ran >= 15, f"only {ran} of 40 random geometries ran on the tensor-core kernels"
