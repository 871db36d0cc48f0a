"""Variable-size batches and extra tokens on the tensor-core kernels: one launch per kernel for the whole
batch (every sample has TMA tensor maps with its own bounds; tiles outside a sample are skipped), the extra
tokens as one more chunk of keys of the same softmax and as extra work items of the dK/dV kernel.

Padding is filled with NaN on purpose: the reference slices every sample out of the padded
tensors (src/natten_mlx/_core/pure.py:559-577), so nothing outside a sample's extents may reach
the arithmetic, and the padding of outputs and gradients must come back as exact zeros
(tests/test_varlen_na2d.py:118-131, 235-252).  Compared with the CPU oracle (bf16: 2e-2 of the
largest magnitude) for 1-D/2-D/3-D, GQA, dilation, with and without extra tokens and LSE."""

from __future__ import annotations

import pytest
import torch

import natten_oracle as oracle

import natten_mlx_b200 as nb
from natten_mlx_b200 import _lib
from natten_mlx_b200._core import cuda as backend

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(shape, seed, dtype=torch.float32):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(dtype)


def _poison(t, sizes):
    """NaN outside each sample's extents."""
    t = t.clone()
    rank = len(sizes[0])
    for b, size in enumerate(sizes):
        keep = torch.zeros(t.shape[1:1 + rank], dtype=torch.bool)
        keep[tuple(slice(0, s) for s in size)] = True
        t[b][~keep] = float("nan")
    return t


def _close(got, want, name):
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert torch.isfinite(got).all(), name
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-6))
    assert err < 2e-2, (name, err)


CASES = [
    # padded shape [B, spatial..., Hq, D], kv heads, sizes, kernel, dilation, extra tokens
    ((3, 40, 4, 32), 2, [(40,), (17,), (26,)], (7,), (2,), 0),
    ((3, 24, 20, 4, 32), 4, [(24, 20), (9, 13), (16, 8)], (5, 7), (1, 1), 0),
    ((2, 26, 30, 8, 64), 2, [(26, 22), (18, 30)], (3, 5), (2, 3), 5),
    ((2, 6, 12, 10, 2, 32), 2, [(6, 12, 10), (4, 7, 9)], (3, 3, 5), (1, 2, 1), 3),
]


@pytest.mark.parametrize("shape,hkv,sizes,ks,dl,n_extra", CASES)
def test_tensor_core_varlen_one_launch_per_kernel(shape, hkv, sizes, ks, dl, n_extra):
    rank = len(shape) - 3
    dt = torch.bfloat16
    kv_shape = shape[:-2] + (hkv, shape[-1])
    q, k, v = _rand(shape, 1, dt), _rand(kv_shape, 2, dt), _rand(kv_shape, 3, dt)
    cot, cot_l = _rand(shape, 4, dt), _rand(shape[:-1], 5)
    ak = av = None
    if n_extra:
        ak, av = _rand((shape[0], n_extra, hkv, shape[-1]), 6, dt), _rand((shape[0], n_extra, hkv, shape[-1]), 7, dt)
    ins = [q, k, v] + ([ak, av] if n_extra else [])
    sz = [s[0] for s in sizes] if rank == 1 else sizes

    def ref(*t):
        return oracle.na_varlen(t[0], t[1], t[2], sz, ks if rank > 1 else ks[0], dl if rank > 1 else dl[0],
                                return_lse=True, additional_keys=t[3] if n_extra else None,
                                additional_values=t[4] if n_extra else None)
    (o_ref, l_ref), g_ref = oracle.grads(ref, [t.float() for t in ins], (cot.float(), cot_l))

    st = torch.tensor(sz, dtype=torch.int32, device=DEV)
    fn = {1: nb.na1d_varlen, 2: nb.na2d_varlen, 3: nb.na3d_varlen}[rank]
    dev_ins = [_poison(t, sizes).to(DEV).requires_grad_(True) for t in ins[:3]] + \
              [t.to(DEV).requires_grad_(True) for t in ins[3:]]
    n0 = _lib.launch_count()
    out, lse = fn(dev_ins[0], dev_ins[1], dev_ins[2], st, ks if rank > 1 else ks[0], dl if rank > 1 else dl[0],
                  return_lse=True, additional_keys=dev_ins[3] if n_extra else None,
                  additional_values=dev_ins[4] if n_extra else None, host_sizes=sz)
    assert _lib.last_path() == "tcgen05" and _lib.kernel_status() == 0
    n1 = _lib.launch_count()
    assert n1 - n0 == 1, "the forward of a variable-size batch is one launch"
    grads = torch.autograd.grad((out, lse), dev_ins, (_poison(cot, sizes).to(DEV).nan_to_num(0.0), cot_l.to(DEV)))
    # pre-pass, dQ, dK/dV (+ one cast of the extra-token accumulators)
    assert _lib.launch_count() - n1 == (4 if n_extra else 3) and _lib.kernel_status() == 0
    _close(out, o_ref, "out")
    _close(lse, l_ref, "lse")
    for name, a, b in zip(("dq", "dk", "dv", "dak", "dav"), grads, g_ref):
        _close(a, b, name)
    # padding is exactly zero in outputs and gradients
    for b, size in enumerate(sizes):
        keep = torch.zeros(shape[1:1 + rank], dtype=torch.bool)
        keep[tuple(slice(0, s) for s in size)] = True
        for t in (out, lse) + tuple(grads[:3]):
            assert float(t[b][~keep.to(DEV)].detach().abs().sum()) == 0.0


def test_mem_extent_is_refused_where_it_does_not_apply():
    g = _lib.make_geom(1, 1, 2, 2, 32, _lib.F32, [16], [3], [1], [1], [0], 1.0, mem_extent=[32])
    lib = _lib.load()
    assert lib.natten_b200_fused_forward(g, *([None] * 8)) == _lib.EINVAL          # null tensors are reported first
    q = torch.zeros(1, 32, 2, 32, device=DEV)
    o, l = torch.zeros_like(q), torch.zeros(1, 32, 2, device=DEV)
    rc = lib.natten_b200_fused_forward(g, q.data_ptr(), q.data_ptr(), q.data_ptr(), None, None, o.data_ptr(),
                                       l.data_ptr(), None)
    assert rc == _lib.EINVAL and "tensor-core" in _lib.last_error()                 # float32 has no tensor-core plan
    g2 = _lib.make_geom(1, 1, 2, 2, 32, _lib.BF16, [16], [3], [1], [1], [0], 1.0, mem_extent=[8])
    assert lib.natten_b200_fused_forward(g2, q.data_ptr(), q.data_ptr(), q.data_ptr(), None, None, o.data_ptr(),
                                         l.data_ptr(), None) == _lib.EINVAL
    assert "smaller" in _lib.last_error()
    assert lib.natten_b200_qk_forward(_lib.make_geom(1, 1, 2, 2, 32, _lib.BF16, [16], [3], [1], [1], [0], 1.0,
                                                     mem_extent=[32]), q.data_ptr(), q.data_ptr(), None, o.data_ptr(),
                                      None) == _lib.EINVAL


@pytest.mark.parametrize("shape,hkv,ks,dl,ca,n_extra", [
    ((2, 20, 24, 4, 64), 2, (7, 5), (1, 2), (False, False), 6),
    ((1, 40, 2, 32), 2, (9,), (1,), (True,), 3),
    ((1, 12, 14, 8, 32), 2, (5, 5), (1, 1), (False, False), 150),      # more extra tokens than a tile of 128 rows
    ((2, 4, 10, 12, 2, 64), 1, (3, 5, 3), (1, 1, 2), (True, False, False), 20),
])
def test_extra_tokens_inside_the_tensor_core_kernels(shape, hkv, ks, dl, ca, n_extra):
    """Dense (not variable-size) call with extra tokens in bf16: window and extra tokens share the softmax of
    the tensor-core kernels; out, lse and all gradients (including the one that flows through the returned
    lse) against the oracle."""
    rank = len(shape) - 3
    dt = torch.bfloat16
    kv_shape = shape[:-2] + (hkv, shape[-1])
    ins = [_rand(shape, 1, dt), _rand(kv_shape, 2, dt), _rand(kv_shape, 3, dt),
           _rand((shape[0], n_extra, hkv, shape[-1]), 6, dt), _rand((shape[0], n_extra, hkv, shape[-1]), 7, dt)]
    cot, cot_l = _rand(shape, 4, dt), _rand(shape[:-1], 5)
    ref = lambda q, k, v, a, b: oracle.na(q, k, v, ks, 1, dl, ca, return_lse=True, additional_keys=a,
                                          additional_values=b)
    (o_ref, l_ref), g_ref = oracle.grads(ref, [t.float() for t in ins], (cot.float(), cot_l))
    fn = {1: nb.na1d, 2: nb.na2d, 3: nb.na3d}[rank]
    dev_ins = [t.to(DEV).requires_grad_(True) for t in ins]
    n0 = _lib.launch_count()
    out, lse = fn(dev_ins[0], dev_ins[1], dev_ins[2], kernel_size=ks, dilation=dl, is_causal=ca, return_lse=True,
                  additional_keys=dev_ins[3], additional_values=dev_ins[4])
    assert _lib.last_path() == "tcgen05" and _lib.launch_count() - n0 == 1
    grads = torch.autograd.grad((out, lse), dev_ins, (cot.to(DEV), cot_l.to(DEV)))
    _close(out, o_ref, "out")
    _close(lse, l_ref, "lse")
    for name, a, b in zip(("dq", "dk", "dv", "dak", "dav"), grads, g_ref):
        _close(a, b, name)
