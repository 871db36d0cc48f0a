"""The tensor-core (tcgen05 / TMEM / TMA) fused kernels against the CPU oracle
and against the CUDA-core kernels, through the C ABI with the kernel family
forced.  bf16 / fp16 tolerance against the float32 oracle: 2e-2 of the largest reference
magnitude and 5e-2 per element (|err| <= 5e-2 * (|ref| + rms(ref)))."""

from __future__ import annotations

import pytest
import torch

import natten_oracle as oracle
from conftest import assert_lowp, lowp_errors

from natten_mlx_b200 import _lib
from natten_mlx_b200._core import cuda as backend

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(shape, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype)


def _rel(got, want):
    """Max-norm relative error (used between two low-precision results)."""
    return lowp_errors(got, want)["maxnorm"]


def _check(got, want, name, rel=2e-2):
    """Against the float32 oracle: max-norm and per-element criterion, observed errors recorded."""
    assert_lowp(got, want, name, rel)


CASES = [
    # shape [B, spatial..., Hq, D], heads_kv, kernel, dilation, causal
    ((1, 16, 8, 1, 32), 1, (3, 3), (1, 1), (False, False)),          # one tile, one chunk
    ((2, 56, 56, 4, 32), 4, (7, 7), (1, 1), (False, False)),         # the NAT-stage shape
    ((1, 56, 56, 2, 32), 2, (7, 7), (4, 4), (False, False)),         # 16 dilation classes
    ((1, 30, 23, 2, 32), 2, (5, 7), (2, 3), (True, False)),          # ragged classes, causal axis
    ((2, 150, 4, 32), 4, (7,), (1,), (False,)),                      # 1D
    ((1, 300, 2, 64), 2, (31,), (2,), (True,)),                      # 1D causal, D=64
    ((1, 20, 24, 2, 64), 2, (7, 7), (1, 2), (False, False)),         # D=64 (128-byte swizzle)
    ((1, 18, 20, 2, 128), 2, (5, 5), (1, 1), (False, False)),        # D=128 (two 64-wide blocks)
    ((1, 6, 16, 18, 2, 64), 2, (3, 7, 7), (1, 2, 2), (True, False, False)),   # 3D, several chunks
    ((1, 5, 9, 12, 2, 32), 2, (3, 3, 5), (1, 1, 1), (False, False, False)),
    ((1, 20, 22, 8, 128), 2, (13, 13), (1, 1), (False, False)),      # GQA: 4 query heads packed per tile
    ((1, 12, 14, 4, 32), 2, (4, 6), (1, 1), (False, False)),         # even kernels
    ((1, 24, 20, 4, 32), 4, (5, 7), (1, 1), (False, False)),         # key tiles narrower than the kernel (4 < 5)
    ((1, 30, 23, 2, 32), 2, (7, 5), (1, 2), (False, False)),
    ((8, 64, 64, 8, 32), 8, (3, 3), (1, 1), (False, False)),         # 2048 tiles: every CTA walks several tiles
    ((6, 48, 40, 8, 64), 2, (5, 3), (2, 1), (False, True)),          # several tiles per CTA with packed heads
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,hkv,ks,dl,ca", CASES)
def test_tcgen05_forward(dtype, shape, hkv, ks, dl, ca):
    rank = len(shape) - 3
    kv_shape = shape[:-2] + (hkv, shape[-1])
    q, k, v = _rand(shape, 1, dtype), _rand(kv_shape, 2, dtype), _rand(kv_shape, 3, dtype)
    one = (1,) * rank
    o_ref, l_ref = oracle.na(q.float(), k.float(), v.float(), ks, 1, dl, ca, return_lse=True)
    out, lse = backend.fused_forward(q.to(DEV), k.to(DEV), v.to(DEV), ks, one, dl, ca, None, path="tcgen05")
    torch.cuda.synchronize()
    assert _lib.last_path() == "tcgen05"
    assert _lib.kernel_status() == 0, "a tensor-core kernel gave up on a wait"
    assert out.dtype == dtype and lse.dtype == torch.float32
    _check(out, o_ref, "out")
    _check(lse, l_ref, "lse")
    # and against the CUDA-core kernels on the same inputs
    out_s, lse_s = backend.fused_forward(q.to(DEV), k.to(DEV), v.to(DEV), ks, one, dl, ca, None, path="simt")
    assert _rel(out, out_s) < 2e-2
    assert _rel(lse, lse_s) < 5e-3


def test_tcgen05_is_refused_for_unsupported_shapes():
    q = torch.randn(1, 16, 2, 12, device=DEV)
    with pytest.raises(ValueError, match="tcgen05"):
        backend.fused_forward(q, q, q, (3,), (1,), (1,), (False,), None, path="tcgen05")
    q = torch.randn(1, 16, 2, 32, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="stride and dilation"):
        backend.fused_forward(q, q, q, (3,), (2,), (2,), (False,), None, path="tcgen05")


STRIDED = [
    # shape, heads_kv, kernel, stride, dilation, causal
    ((2, 30, 23, 2, 32), 2, (5, 7), (2, 3), (1, 1), (False, False)),
    ((1, 24, 28, 4, 64), 2, (3, 5), (2, 1), (1, 2), (False, True)),       # a strided axis beside a dilated one; GQA
    ((2, 150, 4, 32), 4, (7,), (2,), (1,), (False,)),
    ((1, 57, 2, 64), 2, (9,), (4,), (1,), (True,)),
    ((1, 6, 13, 12, 2, 32), 2, (3, 5, 3), (1, 2, 2), (1, 1, 1), (True, False, False)),
    ((2, 56, 56, 4, 32), 4, (7, 7), (2, 2), (1, 1), (False, False)),      # several tiles per CTA
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,hkv,ks,st,dl,ca", STRIDED)
def test_tcgen05_strided_forward_backward(dtype, shape, hkv, ks, st, dl, ca):
    """Queries on a stride lattice on the tensor-core kernels (src/natten_mlx/_core/pure.py:19-21): out, lse and
    all gradients against the oracle; dQ rows off the lattice are exact zeros."""
    rank = len(shape) - 3
    kv_shape = shape[:-2] + (hkv, shape[-1])
    q, k, v = _rand(shape, 1, dtype), _rand(kv_shape, 2, dtype), _rand(kv_shape, 3, dtype)
    outs = tuple(-(-shape[1 + a] // st[a]) for a in range(rank))
    cot = _rand((shape[0],) + outs + shape[-2:], 4, dtype)
    cot_l = _rand((shape[0],) + outs + (shape[-2],), 5, torch.float32)
    fn = lambda a, b, c: oracle.na(a, b, c, ks, st, dl, ca, return_lse=True)
    (o_ref, l_ref), g_ref = oracle.grads(fn, [q.float(), k.float(), v.float()], (cot.float(), cot_l))
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out, lse = backend.fused_forward(qd, kd, vd, ks, st, dl, ca, None, path="tcgen05")
    dq, dk, dv, _, _ = backend.fused_backward(qd, kd, vd, out, lse, cot.to(DEV), cot_l.to(DEV), ks, st, dl, ca, None,
                                              path="tcgen05")
    torch.cuda.synchronize()
    assert _lib.last_path() == "tcgen05" and _lib.kernel_status() == 0
    _check(out, o_ref, "out")
    _check(lse, l_ref, "lse")
    for name, got, want in zip(("dq", "dk", "dv"), (dq, dk, dv), g_ref):
        _check(got, want, name)
    on = torch.zeros(shape[1:1 + rank], dtype=torch.bool)
    on[tuple(slice(0, None, s_) for s_ in st)] = True
    assert float(dq[:, ~on.to(DEV)].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,hkv,ks,dl,ca", CASES)
def test_tcgen05_backward(dtype, shape, hkv, ks, dl, ca):
    rank = len(shape) - 3
    kv_shape = shape[:-2] + (hkv, shape[-1])
    q, k, v = _rand(shape, 1, dtype), _rand(kv_shape, 2, dtype), _rand(kv_shape, 3, dtype)
    cot, cot_l = _rand(shape, 4, dtype), _rand(shape[:-1], 5, torch.float32)
    one = (1,) * rank
    fn = lambda a, b, c: oracle.na(a, b, c, ks, 1, dl, ca, return_lse=True)
    _, g_ref = oracle.grads(fn, [q.float(), k.float(), v.float()], (cot.float(), cot_l))
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out, lse = backend.fused_forward(qd, kd, vd, ks, one, dl, ca, None, path="tcgen05")
    dq, dk, dv, _, _ = backend.fused_backward(qd, kd, vd, out, lse, cot.to(DEV), cot_l.to(DEV), ks, one, dl, ca, None,
                                              path="tcgen05")
    torch.cuda.synchronize()
    assert _lib.last_path() == "tcgen05"
    assert _lib.kernel_status() == 0, "a tensor-core kernel gave up on a wait"
    for name, got, want in zip(("dq", "dk", "dv"), (dq, dk, dv), g_ref):
        assert got.dtype == dtype
        _check(got, want, name)
    # bit-identical on a second run (no atomics anywhere)
    dq2, dk2, dv2, _, _ = backend.fused_backward(qd, kd, vd, out, lse, cot.to(DEV), cot_l.to(DEV), ks, one, dl, ca,
                                                 None, path="tcgen05")
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


@pytest.mark.parametrize("shape,ks,dl,ca,world", [
    ((1, 12, 9, 10, 2, 32), (3, 3, 5), (2, 1, 1), (True, False, False), 2),
    ((1, 12, 9, 10, 2, 32), (3, 3, 5), (2, 1, 1), (False, False, False), 2),
    ((2, 16, 12, 16, 4, 64), (5, 7, 3), (1, 1, 2), (False, False, False), 3),
    ((1, 20, 8, 8, 2, 32), (3, 3, 3), (3, 1, 1), (True, False, False), 4),
])
def test_leading_axis_slabs_on_the_tensor_core_kernels(shape, ks, dl, ca, world):
    """Slabs of a 3-D volume along its leading axis (K/V with halo planes, windows in global
    coordinates): out and dq of every slab, and dk/dv with the halo partials added, equal the
    unsharded result of the same kernels."""
    from natten_mlx_b200.sharding import fused_slab_forward_backward, slab_plan
    dt = torch.bfloat16
    q, k, v, cot = (_rand(shape, 100 + i, dt).to(DEV) for i in range(4))
    one = (1, 1, 1)
    o_ref, lse_ref = backend.fused_forward(q, k, v, ks, one, dl, ca, None, path="tcgen05")
    g_ref = backend.fused_backward(q, k, v, o_ref, lse_ref, cot, None, ks, one, dl, ca, None, path="tcgen05")
    T = shape[1]
    dk_full, dv_full = torch.zeros_like(k, dtype=torch.float32), torch.zeros_like(v, dtype=torch.float32)
    for r in range(world):
        plan = slab_plan(T, world, r, ks[0], dl[0], ca[0])
        o, lse, dq, dk_, dv_ = fused_slab_forward_backward(
            q[:, plan.q_lo:plan.q_hi], k[:, plan.kv_lo:plan.kv_hi], v[:, plan.kv_lo:plan.kv_hi],
            cot[:, plan.q_lo:plan.q_hi], plan, shape[1:4], ks, dl, ca, None)
        assert _lib.last_path() == "tcgen05" and _lib.kernel_status() == 0
        assert _rel(o, o_ref[:, plan.q_lo:plan.q_hi]) < 1e-2            # tiles differ, so rounding may
        assert _rel(lse, lse_ref[:, plan.q_lo:plan.q_hi]) < 1e-3
        assert _rel(dq, g_ref[0][:, plan.q_lo:plan.q_hi]) < 1e-2
        dk_full[:, plan.kv_lo:plan.kv_hi] += dk_.float()
        dv_full[:, plan.kv_lo:plan.kv_hi] += dv_.float()
    assert _rel(dk_full, g_ref[1]) < 2e-2
    assert _rel(dv_full, g_ref[2]) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape,ks,dl,ca,world", [
    ((2, 12, 9, 10, 2, 32), (3, 3, 5), (1, 1, 1), (True, False, False), 2),
    ((2, 16, 12, 16, 4, 64), (5, 7, 3), (1, 1, 2), (False, False, False), 3),
])
def test_slab_forward_in_pieces(dtype, shape, ks, dl, ca, world):
    """The forward of a slab launched as interior planes first and boundary planes afterwards, sample by sample
    and into slices of the outputs (what the sharded forward does while the halo planes travel), equals the
    one-launch forward of the slab."""
    from natten_mlx_b200 import sharding
    q, k, v = (_rand(shape, 400 + i, dtype).to(DEV) for i in range(3))
    one = (1, 1, 1)
    for r in range(world):
        plan = sharding.slab_plan(shape[1], world, r, ks[0], dl[0], ca[0])
        below, above, planes = plan.q_lo - plan.kv_lo, plan.kv_hi - plan.q_hi, plan.q_hi - plan.q_lo
        qs = q[:, plan.q_lo:plan.q_hi].contiguous()
        kb, vb = k[:, plan.kv_lo:plan.kv_hi].contiguous(), v[:, plan.kv_lo:plan.kv_hi].contiguous()
        o_ref, l_ref = backend.fused_forward(qs, kb, vb, ks, one, dl, ca, None, slab=sharding._slab(plan, shape[1:4]))
        out = torch.full_like(qs, float("nan"))
        lse = torch.full(qs.shape[:-1], float("nan"), dtype=torch.float32, device=DEV)
        for p0, p1 in ((below, planes - above), (0, below), (planes - above, planes)):
            sharding.slab_forward_planes(qs, kb, vb, out, lse, plan, shape[1:4], ks, dl, ca, None, p0, p1)
        tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
        assert _rel(out, o_ref) < tol and _rel(lse, l_ref) < tol / 10
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("shape,ks,dl,ca,world", [
    ((2, 12, 9, 10, 2, 32), (3, 3, 5), (1, 1, 1), (True, False, False), 2),
    ((2, 16, 12, 16, 4, 64), (5, 7, 3), (1, 1, 2), (False, False, False), 3),
])
def test_dkdv_kernel_delivers_the_gradients_of_halo_planes_elsewhere(shape, ks, dl, ca, world):
    """``halo_out``: the dK/dV kernel stores the gradients of a slab's leading / trailing halo planes into other
    tensors ([batch, planes, ...]; on several GPUs the neighbours' staging areas) and leaves those planes of
    dk / dv alone; everything equals the plain slab backward bit for bit."""
    from natten_mlx_b200 import sharding
    dt = torch.bfloat16
    q, k, v, cot = (_rand(shape, 300 + i, dt).to(DEV) for i in range(4))
    one = (1, 1, 1)
    T = shape[1]
    seen = 0
    for r in range(world):
        plan = sharding.slab_plan(T, world, r, ks[0], dl[0], ca[0])
        below, above = plan.q_lo - plan.kv_lo, plan.kv_hi - plan.q_hi
        slab = sharding._slab(plan, shape[1:4])
        qs, ks_, vs, cs = (t[:, a:b].contiguous() for t, (a, b) in
                           ((q, (plan.q_lo, plan.q_hi)), (k, (plan.kv_lo, plan.kv_hi)), (v, (plan.kv_lo, plan.kv_hi)),
                            (cot, (plan.q_lo, plan.q_hi))))
        o, lse = backend.fused_forward(qs, ks_, vs, ks, one, dl, ca, None, slab=slab, path="tcgen05")
        dq0, dk0, dv0, _, _ = backend.fused_backward(qs, ks_, vs, o, lse, cs, None, ks, one, dl, ca, None, slab=slab,
                                                     path="tcgen05")
        if below + above == 0:
            continue
        seen += 1
        mk = lambda n: torch.full((shape[0], max(n, 1)) + tuple(ks_.shape[2:]), 7.0, dtype=dt, device=DEV)
        kb, vb, ka, va = mk(below), mk(below), mk(above), mk(above)
        halo = (below, above, kb.data_ptr() if below else 0, vb.data_ptr() if below else 0,
                ka.data_ptr() if above else 0, va.data_ptr() if above else 0)
        dq1, dk1, dv1, _, _ = backend.fused_backward(qs, ks_, vs, o, lse, cs, None, ks, one, dl, ca, None, slab=slab,
                                                     path="tcgen05", halo_out=halo)
        torch.cuda.synchronize()
        assert _lib.kernel_status() == 0
        n = ks_.shape[1]
        assert torch.equal(dq1, dq0)
        assert torch.equal(dk1[:, below:n - above], dk0[:, below:n - above])
        assert torch.equal(dv1[:, below:n - above], dv0[:, below:n - above])
        if below:
            assert torch.equal(kb, dk0[:, :below]) and torch.equal(vb, dv0[:, :below])
        if above:
            assert torch.equal(ka, dk0[:, n - above:]) and torch.equal(va, dv0[:, n - above:])
    assert seen >= world - 1
    with pytest.raises(ValueError, match="tensor-core"):        # the float32 kernels have no such output
        f = lambda t: t.float()
        plan = sharding.slab_plan(T, world, 1, ks[0], dl[0], ca[0])
        slab = sharding._slab(plan, shape[1:4])
        qs, ks_, vs = f(q[:, plan.q_lo:plan.q_hi]), f(k[:, plan.kv_lo:plan.kv_hi]), f(v[:, plan.kv_lo:plan.kv_hi])
        o, lse = backend.fused_forward(qs, ks_, vs, ks, one, dl, ca, None, slab=slab)
        backend.fused_backward(qs, ks_, vs, o, lse, f(cot[:, plan.q_lo:plan.q_hi]), None, ks, one, dl, ca, None, slab=slab,
                               halo_out=(1, 0, o.data_ptr(), o.data_ptr(), 0, 0))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_two_devices_in_one_process():
    """The opt-in to large dynamic shared memory belongs to a device's context: the tensor-core kernels must launch
    on a second device of the same process too, and give the same bits there."""
    shape, ks = (1, 24, 20, 4, 32), (7, 5)
    q, k, v = (_rand(shape, 200 + i, torch.bfloat16) for i in range(3))
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        o, lse = backend.fused_forward(q.to(dev), k.to(dev), v.to(dev), ks, (1, 1), (1, 1), (False, False), None,
                                       path="tcgen05")
        g = backend.fused_backward(q.to(dev), k.to(dev), v.to(dev), o, lse, torch.ones_like(o), None, ks, (1, 1), (1, 1),
                                   (False, False), None, path="tcgen05")
        torch.cuda.synchronize(dev)
        with torch.cuda.device(dev):
            assert _lib.kernel_status() == 0
        outs.append([t.cpu() for t in (o, lse) + tuple(g[:3])])
    for a, b in zip(*outs):
        assert torch.equal(a, b)
