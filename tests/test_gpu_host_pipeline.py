"""Host-resident tensors streamed through the GPU in batch slabs (``natten_mlx_b200.host``)
against one call of the device API over the whole batch: the results must be identical bit for
bit, because a slab is a set of whole samples and nothing is reduced across samples."""

from __future__ import annotations

import pytest
import torch

from natten_mlx_b200._core import cuda as backend
from natten_mlx_b200.host import HostPipeline

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("shape,hkv,ks,dl,ca,slabs", [
    ((6, 24, 20, 4, 32), 2, (7, 5), (1, 2), (False, True), 4),      # ragged slabs: 2 + 2 + 2 of 6 -> ceil(6/4)=2
    ((5, 40, 2, 32), 2, (5,), (2,), (False,), 2),                   # 1-D, slabs of 3 and 2
])
def test_host_pipeline_matches_device_call(shape, hkv, ks, dl, ca, slabs):
    gen = torch.Generator().manual_seed(5)
    kv_shape = shape[:-2] + (hkv, shape[-1])
    mk = lambda s: torch.randn(s, generator=gen).to(torch.bfloat16).pin_memory()
    q, k, v, cot = mk(shape), mk(kv_shape), mk(kv_shape), mk(shape)
    outs = [torch.empty_like(t).pin_memory() for t in (q, q, k, v)]
    pipe = HostPipeline(shape, torch.bfloat16, DEV, ks, dilation=dl, is_causal=ca, heads_kv=hkv, slabs=slabs)
    for _ in range(2):                                   # the plan is reusable
        pipe.run(q, k, v, cot, *outs)
        torch.cuda.synchronize()
    one = (1,) * len(ks)
    qd, kd, vd, cd = (t.to(DEV) for t in (q, k, v, cot))
    o, lse = backend.fused_forward(qd, kd, vd, ks, one, dl, ca, None)
    dq, dk, dv, _, _ = backend.fused_backward(qd, kd, vd, o, lse, cd, None, ks, one, dl, ca, None)
    for got, want in zip(outs, (o, dq, dk, dv)):
        assert torch.equal(got, want.cpu())


def test_host_pipeline_rejects_other_shapes():
    pipe = HostPipeline((2, 16, 2, 32), torch.bfloat16, DEV, (3,))
    t = torch.zeros(2, 17, 2, 32, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="shapes"):
        pipe.run(t, t, t, t, t, t, t, t)
