"""Leading-axis sharding: slab plans and the halo exchange, on CPU ranks (gloo).

The exchange code is device-agnostic (torch.distributed point-to-point), so two
CPU processes exercise the same logic the NCCL ranks run.  The attention math
of a slab is checked with the CPU oracle: a rank's output must equal the
unsharded output on its planes when every key plane outside its assembled K/V
buffer is poisoned with NaN, i.e. the buffer holds every key it can address.
"""

from __future__ import annotations

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import natten_oracle as oracle
from natten_mlx_b200 import sharding


def test_slab_plans_cover_every_window():
    for extent, world, K, d, causal in [(32, 8, 3, 1, True), (32, 4, 3, 1, False), (24, 3, 5, 2, False),
                                        (17, 2, 7, 1, False), (40, 4, 4, 3, True), (12, 2, 3, 2, False)]:
        plans = sharding.all_plans(extent, world, K, d, causal)
        assert plans[0].q_lo == 0 and plans[-1].q_hi == extent
        idx, ok = oracle.axis_table(np.arange(extent), extent, K, d, causal)
        for p in plans:
            assert p.q_lo < p.q_hi
            used = idx[p.q_lo:p.q_hi][ok[p.q_lo:p.q_hi]]
            assert p.kv_lo == used.min() and p.kv_hi == used.max() + 1
            if causal:
                assert p.kv_hi == p.q_hi           # nothing is needed from above
        # a causal T axis with K_T=3, dilation 1 borrows exactly two planes from below
        if (K, d, causal) == (3, 1, True):
            assert all(p.q_lo - p.kv_lo == (2 if p.rank else 0) for p in plans)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, extent, K, d, causal, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(5)
        shape = (2, extent, 3, 4, 2, 8)
        k_full = torch.randn(shape, generator=gen)
        g_full = [torch.randn(shape, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
        plans = sharding.all_plans(extent, world, K, d, causal)
        me = plans[rank]
        # forward halo: the assembled buffer equals the global planes [kv_lo, kv_hi)
        buf = sharding.exchange_halo(k_full[:, me.q_lo:me.q_hi].contiguous(), plans, rank)
        ok_fwd = torch.equal(buf, k_full[:, me.kv_lo:me.kv_hi])
        # backward halo: every rank holds a gradient buffer over its [kv_lo, kv_hi); owners sum the partials
        mine = g_full[rank][:, me.kv_lo:me.kv_hi].contiguous()
        own = sharding.reduce_halo_grads(mine, plans, rank)
        want = torch.zeros_like(own)
        for r, p in enumerate(plans):
            lo, hi = max(p.kv_lo, me.q_lo), min(p.kv_hi, me.q_hi)
            if hi > lo:
                want[:, lo - me.q_lo:hi - me.q_lo] += g_full[r][:, lo:hi]
        ok_bwd = torch.allclose(own, want, atol=1e-6)
        # the buffer holds every key the slab's queries address (oracle with poisoned planes)
        q_full = torch.randn((1, extent, 4, 5, 2, 8), generator=gen)
        kk = torch.randn((1, extent, 4, 5, 2, 8), generator=gen)
        ks, dl, ca = (K, 3, 3), (d, 1, 1), (causal, False, False)
        ref = oracle.na(q_full, kk, kk, ks, 1, dl, ca)
        poisoned = kk.clone()
        poisoned[:, :me.kv_lo] = float("nan")
        poisoned[:, me.kv_hi:] = float("nan")
        got = oracle.na(q_full, poisoned, poisoned, ks, 1, dl, ca)[:, me.q_lo:me.q_hi]
        ok_cover = torch.allclose(got, ref[:, me.q_lo:me.q_hi], atol=1e-6, equal_nan=False)
        results[rank] = (ok_fwd, ok_bwd, ok_cover)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("extent,K,d,causal", [(12, 3, 1, True), (12, 3, 2, False), (11, 5, 1, False)])
def test_halo_exchange_two_ranks(extent, K, d, causal):
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = _free_port()
    mp.spawn(_worker, args=(world, port, extent, K, d, causal, results), nprocs=world, join=True)
    assert len(results) == world
    for r in range(world):
        assert results[r] == (True, True, True), (r, results[r])
