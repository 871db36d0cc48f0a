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


class _HostPeers:
    """Stands in for ``sharding.PeerTransport`` on the CPU: the ranks' allocations are host tensors of one
    process, the copy is a pitched memmove, the barriers only count (the ranks run one after the other)."""

    def __init__(self, world):
        self.world, self.allocs, self.rank, self.copies, self.epoch, self.barriers = world, {}, 0, 0, 0, 0
        self._pool = {}

    def barrier(self):
        self.epoch += 1
        self.barriers += 1

    def acquire(self, nbytes):
        if nbytes not in self.allocs:
            self.allocs[nbytes] = [torch.zeros(nbytes + 16, dtype=torch.uint8) for _ in range(self.world)]
        tensors = [t[(-t.data_ptr()) % 16:][:nbytes] for t in self.allocs[nbytes]]
        lease = sharding._Lease(self, nbytes, tensors[self.rank], [t.data_ptr() for t in tensors])
        lease.keep = tensors
        return lease

    def copy2d(self, dst, dst_pitch, src, src_pitch, width, rows, dma=False):
        import ctypes
        assert width % 16 == 0 and dst % 16 == 0 and src % 16 == 0
        for r in range(rows):
            ctypes.memmove(dst + r * dst_pitch, src + r * src_pitch, width)
        self.copies += 1


@pytest.mark.parametrize("extent,world,K,d,causal", [(12, 2, 3, 1, True), (12, 4, 3, 2, False), (11, 3, 5, 1, False),
                                                      (32, 8, 3, 1, True), (9, 4, 7, 1, False)])
def test_peer_memory_transport_addressing(monkeypatch, extent, world, K, d, causal):
    """The address arithmetic of the peer-memory exchange (which plane goes where in whose buffer, pitches,
    staging offsets of the gradient partials), run on host memory for every rank in turn."""
    plans = sharding.all_plans(extent, world, K, d, causal)
    transfers = sharding.halo_transfers(plans)
    for p in plans:                                  # the transfers cover every borrowed plane exactly once
        got = sorted(x for o, b, lo, hi in transfers if b == p.rank for x in range(lo, hi))
        assert got == [x for x in range(p.kv_lo, p.kv_hi) if not p.q_lo <= x < p.q_hi]
    where, span = sharding.staging_layout(plans)
    for p in plans:                                  # staging ranges of one owner do not overlap
        taken = sorted((where[(o, b)], where[(o, b)] + hi - lo) for o, b, lo, hi in transfers if o == p.rank)
        assert all(a[1] <= b[0] for a, b in zip(taken, taken[1:])) and (not taken or taken[-1][1] <= span)

    peers = _HostPeers(world)
    monkeypatch.setattr(sharding, "peer_transport", lambda group=None: peers)
    gen = torch.Generator().manual_seed(9)
    shape = (2, extent, 3, 2, 8)
    k_full, v_full = torch.randn(shape, generator=gen), torch.randn(shape, generator=gen)
    bufs = {}
    for r, me in enumerate(plans):
        peers.rank = r
        (kb, vb), lease = sharding.exchange_halos_peer([k_full[:, me.q_lo:me.q_hi], v_full[:, me.q_lo:me.q_hi]], plans, r)
        bufs[r] = (kb, vb, lease)
    for r, me in enumerate(plans):                   # after every rank has written: each buffer is the global range
        assert torch.equal(bufs[r][0], k_full[:, me.kv_lo:me.kv_hi])
        assert torch.equal(bufs[r][1], v_full[:, me.kv_lo:me.kv_hi])
    # K/V produced straight into buffers of the allocation: same result, and the owned planes are not copied
    own = {}
    for r, me in enumerate(plans):
        peers.rank = r
        (k_own, v_own), lease = sharding.peer_kv_buffers((2, me.q_hi - me.q_lo, 3, 2, 8), torch.float32, plans, r)
        k_own.copy_(k_full[:, me.q_lo:me.q_hi])
        v_own.copy_(v_full[:, me.q_lo:me.q_hi])
        own[r] = (k_own, v_own, lease)
    for r, me in enumerate(plans):
        peers.rank = r
        (kb, vb), lease = sharding.exchange_halos_peer(own[r][:2], plans, r)
        assert lease is own[r][2] and kb.data_ptr() <= own[r][0].data_ptr()
        bufs[r] = (kb, vb, lease)
    for r, me in enumerate(plans):
        assert torch.equal(bufs[r][0], k_full[:, me.kv_lo:me.kv_hi])
        assert torch.equal(bufs[r][1], v_full[:, me.kv_lo:me.kv_hi])
        own[r][2].release()
    assert not sharding._kv_registry
    # gradients: every rank's buffer over [kv_lo, kv_hi); owners end with the sum of all partials for their planes.
    # The owners add after all ranks have written, so the writes run first and the adds are replayed afterwards.
    grads = [torch.randn(shape, generator=torch.Generator().manual_seed(50 + r)) for r in range(world)]
    mine = [grads[r][:, p.kv_lo:p.kv_hi].contiguous() for r, p in enumerate(plans)]
    for phase in (0, 1):
        for r, me in enumerate(plans):
            peers.rank = r
            if phase == 0:
                saved = mine[r].clone()
                sharding.reduce_halo_grads_peer([mine[r]], plans, r)    # writes the partials (and adds what is there so far)
                mine[r].copy_(saved)
            else:
                own = sharding.reduce_halo_grads_peer([mine[r]], plans, r)[0]
                want = torch.zeros_like(own)
                for o, p in enumerate(plans):
                    lo, hi = max(p.kv_lo, me.q_lo), min(p.kv_hi, me.q_hi)
                    if hi > lo:
                        want[:, lo - me.q_lo:hi - me.q_lo] += grads[o][:, lo:hi]
                assert torch.allclose(own, want, atol=1e-6)


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


def test_lease_asks_for_a_barrier_only_when_none_was_queued_since_the_last_read():
    peers = _HostPeers(2)
    lease = peers.acquire(64)
    assert not lease.needs_barrier()          # fresh memory: nobody has read it
    peers.barrier()
    lease.mark_read()                         # a kernel reading it was queued after barrier 1
    assert lease.needs_barrier()              # a neighbour must not write before another barrier
    peers.barrier()
    assert not lease.needs_barrier()
    lease.mark_read()
    lease.release()
    again = sharding._Lease(peers, 64, *peers._pool[64].pop())
    assert again.needs_barrier()              # the pool remembers when the allocation was last read
    peers.barrier()
    assert not again.needs_barrier()


def test_variable_size_batches_are_balanced_by_tokens():
    sizes = [(104, 96), (112, 128), (112, 88), (88, 88), (120, 88), (64, 88), (72, 128), (96, 64), (72, 72), (72, 80),
             (112, 104), (64, 128), (88, 88), (120, 64), (88, 128), (120, 88)]
    total = sum(h * w for h, w in sizes)
    for world in (1, 2, 4, 8):
        parts = sharding.balance_by_tokens(sizes, world)
        assert sorted(i for p in parts for i in p) == list(range(len(sizes)))
        loads = [sum(sizes[i][0] * sizes[i][1] for i in p) for p in parts]
        assert max(loads) <= 1.1 * total / world + max(h * w for h, w in sizes) * (world > 4)
        by_count = [sum(h * w for h, w in sizes[r::world]) for r in range(world)]
        assert max(loads) <= max(by_count)
    assert sharding.balance_by_tokens([5, 1, 1, 1, 1, 1], 2) == [[0], [1, 2, 3, 4, 5]]
