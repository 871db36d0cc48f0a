"""Leading-axis sharding with the K/V halo exchange on real GPUs, over both transports (the
library's copy kernel writing into the neighbour's symmetric memory, and NCCL point-to-point):
every rank holds its planes of a 3-D volume, calls ``sharding.na_sharded`` forward and
backward, and its planes of the output and of dq/dk/dv must equal the unsharded result of the
same kernels on one GPU.  Needs two or more GPUs; on a single-GPU box the test is skipped (the
same logic runs among CPU ranks in tests/test_sharding_gloo.py and as a one-GPU slab emulation
in tests/test_gpu_parity.py)."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, causal, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import natten_mlx_b200 as nb
        from natten_mlx_b200 import _lib, sharding
        T, ks, dl, ca = 12, (3, 3, 5), (2, 1, 1), (causal, False, False)
        gen = torch.Generator().manual_seed(21)
        full = [torch.randn((2, T, 6, 9, 2, 16), generator=gen) for _ in range(4)]      # q, k, v, cotangent (two samples: halo planes travel per sample)
        bounds = sharding.shard_bounds(T, world)
        lo, hi = bounds[rank], bounds[rank + 1]
        dev = torch.device("cuda", rank)
        # the unsharded result on this rank's GPU
        qf, kf, vf = (t.to(dev).requires_grad_(True) for t in full[:3])
        ref = nb.na3d(qf, kf, vf, kernel_size=ks, dilation=dl, is_causal=ca)
        ref.backward(full[3].to(dev))
        ok = []
        # the peer transport twice: the second step reuses the pooled buffers and the next barrier epochs
        for transport in ("peer", "peer", "p2p"):
            q, k, v = (t[:, lo:hi].to(dev).requires_grad_(True) for t in full[:3])
            out = sharding.na_sharded(q, k, v, T, ks, dl, ca, transport=transport)
            out.backward(full[3][:, lo:hi].to(dev))
            ok.append(torch.allclose(out, ref[:, lo:hi], atol=1e-5, rtol=1e-5))
            for a, b in ((q, qf), (k, kf), (v, vf)):
                ok.append(torch.allclose(a.grad, b.grad[:, lo:hi], atol=1e-4, rtol=1e-4))
        # K and V produced straight into symmetric memory (no copy of the owned planes), two steps
        plans = sharding.all_plans(T, world, ks[0], dl[0], ca[0])
        (kp, vp), kv_lease = sharding.peer_kv_buffers((2, hi - lo, 6, 9, 2, 16), torch.float32, plans, rank)
        kp.copy_(full[1][:, lo:hi])
        vp.copy_(full[2][:, lo:hi])
        kp.requires_grad_(True)
        vp.requires_grad_(True)
        for _ in range(2):
            q = full[0][:, lo:hi].to(dev).requires_grad_(True)
            out = sharding.na_sharded(q, kp, vp, T, ks, dl, ca, transport="peer")
            gq, gk, gv = torch.autograd.grad(out, (q, kp, vp), full[3][:, lo:hi].to(dev))
            ok.append(torch.allclose(out, ref[:, lo:hi], atol=1e-5, rtol=1e-5))
            for a, b in ((gq, qf), (gk, kf), (gv, vf)):
                ok.append(torch.allclose(a, b.grad[:, lo:hi], atol=1e-4, rtol=1e-4))
        kv_lease.release()
        ok.append(_lib.kernel_status() == 0)          # no barrier gave up on its wait
        # bf16 on the tensor-core kernels: the dK/dV kernel itself delivers the halo planes' gradients into the
        # neighbours' staging areas (no copy kernel in the backward)
        bf = torch.bfloat16
        gen = torch.Generator().manual_seed(33)
        full16 = [torch.randn((2, T, 10, 16, 2, 32), generator=gen).to(bf) for _ in range(4)]
        ks16, dl16 = (3, 3, 5), (1, 1, 2)
        qf, kf, vf = (t.to(dev).requires_grad_(True) for t in full16[:3])
        ref16 = nb.na3d(qf, kf, vf, kernel_size=ks16, dilation=dl16, is_causal=ca)
        ref16.backward(full16[3].to(dev))
        tc = _lib.last_path() == "tcgen05"
        rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max())
        for _ in range(2):
            q, k, v = (t[:, lo:hi].to(dev).requires_grad_(True) for t in full16[:3])
            out = sharding.na_sharded(q, k, v, T, ks16, dl16, ca, transport="peer")
            _lib.trace_report()
            _lib.trace_enable(True)
            out.backward(full16[3][:, lo:hi].to(dev))
            torch.cuda.synchronize()
            _lib.trace_enable(False)
            names = set(_lib.trace_report())
            ok.append(tc and "fna_bwd_dkv_sm100" in names and "peer_copy2d" not in names and "peer_barrier" in names)
            ok.append(rel(out, ref16[:, lo:hi]) < 2e-2)
            for a, b in ((q, qf), (k, kf), (v, vf)):
                ok.append(rel(a.grad, b.grad[:, lo:hi]) < 2e-2)
        ok.append(_lib.kernel_status() == 0)
        with torch.no_grad():                          # nothing saved: the buffers go straight back to the pool
            q, k, v = (t[:, lo:hi].to(dev) for t in full[:3])
            ok.append(torch.allclose(sharding.na_sharded(q, k, v, T, ks, dl, ca, transport="peer"), ref[:, lo:hi],
                                     atol=1e-5, rtol=1e-5))
        ok.append(len(sharding.peer_transport()._pool) > 0)
        results[rank] = tuple(bool(x) for x in ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("causal", [True, False])
def test_na_sharded_matches_unsharded_over_nccl(causal):
    world = min(torch.cuda.device_count(), 4)
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), causal, results), nprocs=world, join=True)
    assert len(results) == world
    for r in range(world):
        assert all(results[r]) and len(results[r]) == 34, (r, results[r])
