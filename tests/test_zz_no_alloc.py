"""The allocation-free fused backward (``natten_b200_fused_backward_static_scratch``).

A host that may not allocate device memory where the backward runs (its
allocator is frozen while an execution plan is recorded or replayed, or it only
owns pre-registered buffers) passes inputs and outputs and nothing else; the
library's built-in scratch array stands in for the caller-provided scratch
buffer.  The test drives both entry points through the C ABI with the same
device buffers and expects the same gradients, twice in a row (the array keeps
the previous call's contents, so the second call also shows that stale contents
do no harm).  It is collected last on purpose.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from natten_mlx_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _case(dtype, shape, hkv, ks, dl, ca, n_extra, path):
    rank = len(shape) - 3
    gen = torch.Generator().manual_seed(77)
    kv_shape = shape[:-2] + (hkv, shape[-1])
    mk = lambda s: torch.randn(s, generator=gen).to(dtype).to(DEV)
    q, k, v, dout = mk(shape), mk(kv_shape), mk(kv_shape), mk(shape)
    dlse = torch.randn(shape[:-1], generator=gen).to(DEV)
    ke = ve = None
    if n_extra:
        ke, ve = mk((shape[0], n_extra, hkv, shape[-1])), mk((shape[0], n_extra, hkv, shape[-1]))
    code = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}[dtype]
    geom = _lib.make_geom(rank, shape[0], shape[-2], hkv, shape[-1], code, shape[1:1 + rank], ks, [1] * rank, dl,
                          [int(c) for c in ca], shape[-1] ** -0.5, n_extra=n_extra, path=path)
    lib = _lib.load()
    out = torch.empty_like(q)
    lse = torch.empty(shape[:-1], dtype=torch.float32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.natten_b200_fused_forward(geom, _ptr(q), _ptr(k), _ptr(v), _ptr(ke), _ptr(ve), _ptr(out), _ptr(lse),
                                             stream))

    def grads(static, outputs=None):
        if outputs is None:
            outputs = (torch.full_like(q, 7.0), torch.full_like(k, 7.0), torch.full_like(v, 7.0),
                       None if ke is None else torch.full_like(ke, 7.0), None if ve is None else torch.full_like(ve, 7.0))
        dq, dk, dv, dke, dve = outputs
        args = [geom, _ptr(q), _ptr(k), _ptr(v), _ptr(ke), _ptr(ve), _ptr(out), _ptr(lse), _ptr(dout), _ptr(dlse),
                _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dke), _ptr(dve)]
        if static:
            _lib.check(lib.natten_b200_fused_backward_static_scratch(*args, stream))
        else:
            nbytes = int(lib.natten_b200_fused_backward_scratch_bytes(geom))
            scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
            _lib.check(lib.natten_b200_fused_backward(*args, _ptr(scratch), nbytes, stream))
        torch.cuda.synchronize()
        return [t for t in (dq, dk, dv, dke, dve) if t is not None]

    return grads


@pytest.mark.parametrize("dtype,shape,hkv,ks,dl,ca,n_extra,path", [
    (torch.bfloat16, (2, 24, 20, 4, 32), 2, (7, 5), (1, 2), (False, True), 0, _lib.PATH_AUTO),   # tensor-core kernels
    (torch.float32, (2, 40, 4, 16), 4, (5,), (2,), (False,), 3, _lib.PATH_SIMT),                 # CUDA-core kernels + extra tokens
])
def test_static_scratch_backward_matches_regular_entry_point(dtype, shape, hkv, ks, dl, ca, n_extra, path):
    grads = _case(dtype, shape, hkv, ks, dl, ca, n_extra, path)
    want = grads(static=False)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for attempt in range(2):                       # two calls in a row share the built-in array
        got = grads(static=True)
        for a, b in zip(got, want):
            err = (a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6)
            assert err <= tol, (attempt, float(err))
    assert _lib.kernel_status() == 0
    # The entry point's one promise: with the outputs already in place, a call leaves the device's free memory
    # and torch's reserved pool exactly as it found them (the first call on the device, above, did the set-up).
    outputs = tuple(torch.full_like(t, 7.0) for t in want) + (None,) * (5 - len(want))
    torch.cuda.synchronize()
    free_before, reserved_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
    got = grads(static=True, outputs=outputs)
    free_after, reserved_after = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
    assert reserved_after == reserved_before
    assert free_after >= free_before, (free_before, free_after)
    for a, b in zip(got, want):
        assert (a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6) <= tol


def test_static_scratch_refuses_oversized_geometry():
    lib = _lib.load()
    cap = int(lib.natten_b200_static_scratch_capacity())
    assert cap == 4 << 20
    rows_needed = cap // 4 + 1024                     # one float of scratch per (query, head) row
    geom = _lib.make_geom(1, 1, 1, 1, 32, _lib.F32, [rows_needed], [3], [1], [1], [0], 1.0)
    assert int(lib.natten_b200_fused_backward_scratch_bytes(geom)) > cap
    rc = lib.natten_b200_fused_backward_static_scratch(geom, *([None] * 14), None)
    assert rc == _lib.ERESOURCE
    assert "built-in" in _lib.last_error()
