"""Multi-GPU use of the path: batch/head shards need no communication; a large
volume can also be split along its leading spatial axis, with a K/V halo
exchange in the forward and the reverse dK/dV halo reduction in the backward.

The reference is single-device (it has no distributed code); this module is
what makes its operators span the GPUs of one box.  One process per GPU,
``torch.distributed`` point-to-point (NCCL send/recv over NVLink on GPUs, gloo
in the CPU tests).  Halo planes are received into local memory before any
kernel reads them.

Window positions are evaluated in global coordinates: each rank passes its
slab offsets to the kernels (``Slab``), so results equal the unsharded call.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ._core import cuda as _cuda
from .utils import window as _window


@dataclass(frozen=True)
class SlabPlan:
    """Global plane ranges [lo, hi) of one rank along the sharded axis."""
    rank: int
    world: int
    q_lo: int
    q_hi: int
    kv_lo: int   # first plane any local query can address
    kv_hi: int   # one past the last such plane


def shard_bounds(extent: int, world: int) -> List[int]:
    """Balanced contiguous split: rank r owns planes [b[r], b[r+1])."""
    return [(extent * r) // world for r in range(world + 1)]


def slab_plan(extent: int, world: int, rank: int, kernel: int, dilation: int, causal) -> SlabPlan:
    """Which planes rank ``rank`` owns and which K/V planes its queries address.

    The key range is the exact union of the windows of the owned queries,
    evaluated with the library's window table (clamped windows at the volume
    edges need no halo; a causal axis needs none from above)."""
    b = shard_bounds(extent, world)
    q_lo, q_hi = b[rank], b[rank + 1]
    if q_hi <= q_lo:
        raise ValueError(f"rank {rank} of {world} owns no planes of an axis of length {extent}")
    idx, valid, _, _ = _window.axis_table(extent, kernel, dilation, 1, bool(causal))
    rows = slice(q_lo, q_hi)
    used = idx[rows][valid[rows]]
    return SlabPlan(rank, world, q_lo, q_hi, int(used.min()), int(used.max()) + 1)


def all_plans(extent: int, world: int, kernel: int, dilation: int, causal) -> List[SlabPlan]:
    return [slab_plan(extent, world, r, kernel, dilation, causal) for r in range(world)]


def _overlap(a_lo, a_hi, b_lo, b_hi) -> Tuple[int, int]:
    lo, hi = max(a_lo, b_lo), min(a_hi, b_hi)
    return (lo, hi) if hi > lo else (0, 0)


def _planes(t: torch.Tensor, axis: int, lo: int, n: int):
    """Planes [lo, lo + n) of ``t`` along ``axis`` as dense pieces, one per leading index (point-to-point
    transfers need dense tensors).  The split depends on the shape alone, never on whether a particular
    slice happens to be dense, so that sender and receiver always agree on the number of pieces."""
    piece = t.narrow(axis, lo, n)
    lead = list(t.shape[:axis])
    count = 1
    for x in lead:
        count *= x
    if count == 1:
        return [piece.reshape(piece.shape[axis:]) if piece.is_contiguous() else piece.contiguous()]
    flat = piece.reshape([count] + list(piece.shape[axis:])) if len(lead) == 1 else None
    if flat is not None:
        return [flat[i] for i in range(count)]
    out = []
    for idx in torch.cartesian_prod(*[torch.arange(x) for x in lead]).reshape(-1, len(lead)).tolist():
        out.append(piece[tuple(idx)])
    return out


def halo_buffer(local: torch.Tensor, plans: Sequence[SlabPlan], rank: int, axis: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """(buffer over planes [kv_lo, kv_hi), its view of the owned planes [q_lo, q_hi)).  A caller that produces
    its K/V directly into the view saves ``exchange_halo`` the copy of the owned planes."""
    me = plans[rank]
    shape = list(local.shape)
    shape[axis] = me.kv_hi - me.kv_lo
    buf = local.new_empty(shape)
    return buf, buf.narrow(axis, me.q_lo - me.kv_lo, me.q_hi - me.q_lo)


def _is_view_of_own_planes(local: torch.Tensor, me: SlabPlan, axis: int) -> Optional[torch.Tensor]:
    """The halo buffer ``local`` is the owned-planes view of (see ``halo_buffer``), or None."""
    base = local._base
    if base is None or base.dim() != local.dim() or not base.is_contiguous():
        return None
    want = list(local.shape)
    want[axis] = me.kv_hi - me.kv_lo
    if list(base.shape) != want or local.stride() != base.stride():
        return None
    if local.storage_offset() - base.storage_offset() != (me.q_lo - me.kv_lo) * base.stride(axis):
        return None
    return base


def _halo_ops(local, buf, plans, rank, group, axis):
    """Point-to-point operations that fill the halo planes of ``buf`` and lend this rank's planes to the others."""
    me = plans[rank]
    ops = []
    for other in plans:
        if other.rank == rank:
            continue
        lo, hi = _overlap(me.q_lo, me.q_hi, other.kv_lo, other.kv_hi)       # what `other` needs from me
        if hi > lo:
            for piece in _planes(local, axis, lo - me.q_lo, hi - lo):
                ops.append(dist.P2POp(dist.isend, piece, _global_rank(other.rank, group), group))
        lo, hi = _overlap(other.q_lo, other.q_hi, me.kv_lo, me.kv_hi)       # what I need from `other`
        if hi > lo:
            for piece in _planes(buf, axis, lo - me.kv_lo, hi - lo):
                ops.append(dist.P2POp(dist.irecv, piece, _global_rank(other.rank, group), group))
    return ops


def exchange_halos(locals_: Sequence[torch.Tensor], plans: Sequence[SlabPlan], rank: int, group=None,
                   axis: int = 1) -> List[torch.Tensor]:
    """Return, for every tensor of ``locals_`` (K, V, ...), the buffer covering planes [kv_lo, kv_hi) of this rank.

    Each tensor holds the owned planes [q_lo, q_hi) along ``axis``.  Planes owned by other ranks are received
    straight into their place in the buffer; this rank sends the planes others need straight from its tensor
    (no staging copies: transfers go plane range by plane range, per leading index where a range is not
    dense).  A tensor that already is the owned-planes view of a ``halo_buffer`` is not copied at all.  The
    transfers of all tensors travel as one batch.  All ranks must call this in the same order.
    """
    me = plans[rank]
    bufs, ops = [], []
    for local in locals_:
        if me.kv_lo == me.q_lo and me.kv_hi == me.q_hi:
            buf = local if local.is_contiguous() else local.contiguous()   # this rank borrows nothing (it may still lend)
            local = buf
        else:
            buf = _is_view_of_own_planes(local, me, axis)
            if buf is None:
                buf, own = halo_buffer(local, plans, rank, axis)
                own.copy_(local)
        bufs.append(buf)
        ops += _halo_ops(local, buf, plans, rank, group, axis)
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return bufs


def exchange_halo(local: torch.Tensor, plans: Sequence[SlabPlan], rank: int, group=None, axis: int = 1) -> torch.Tensor:
    """``exchange_halos`` for one tensor."""
    return exchange_halos([local], plans, rank, group, axis)[0]


def reduce_halo_grads_many(grad_bufs: Sequence[torch.Tensor], plans: Sequence[SlabPlan], rank: int, group=None,
                           axis: int = 1) -> List[torch.Tensor]:
    """Inverse of ``exchange_halos`` for gradients: every buffer covers planes [kv_lo, kv_hi); partial sums for
    planes owned elsewhere are sent to their owners straight from the buffer, and the owner adds what it receives
    into its planes in place.  Returns the gradients of the owned planes [q_lo, q_hi) (views of the buffers).
    The transfers of all buffers travel as one batch."""
    me = plans[rank]
    owns, ops, recvs = [], [], []
    for grad_buf in grad_bufs:
        own = grad_buf.narrow(axis, me.q_lo - me.kv_lo, me.q_hi - me.q_lo)
        owns.append(own)
        for other in plans:
            if other.rank == rank:
                continue
            lo, hi = _overlap(other.q_lo, other.q_hi, me.kv_lo, me.kv_hi)       # partials I hold for `other`
            if hi > lo:
                for piece in _planes(grad_buf, axis, lo - me.kv_lo, hi - lo):
                    ops.append(dist.P2POp(dist.isend, piece, _global_rank(other.rank, group), group))
            lo, hi = _overlap(me.q_lo, me.q_hi, other.kv_lo, other.kv_hi)       # partials `other` holds for me
            if hi > lo:
                shape = list(own.shape)
                shape[axis] = hi - lo
                piece = own.new_empty(shape)
                recvs.append((own, piece, lo, hi))
                for part in _planes(piece, axis, 0, hi - lo):
                    ops.append(dist.P2POp(dist.irecv, part, _global_rank(other.rank, group), group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    for own, piece, lo, hi in recvs:
        own.narrow(axis, lo - me.q_lo, hi - lo).add_(piece)
    return owns


def reduce_halo_grads(grad_buf: torch.Tensor, plans: Sequence[SlabPlan], rank: int, group=None, axis: int = 1) -> torch.Tensor:
    """``reduce_halo_grads_many`` for one buffer."""
    return reduce_halo_grads_many([grad_buf], plans, rank, group, axis)[0]


def _global_rank(group_rank: int, group) -> int:
    if group is None:
        return group_rank
    return dist.get_global_rank(group, group_rank)


def _slab(plan: SlabPlan, extent: Sequence[int]) -> _cuda.Slab:
    rank = len(extent)
    return _cuda.Slab(tuple(extent), (plan.q_lo,) + (0,) * (rank - 1), (plan.kv_lo,) + (0,) * (rank - 1))


def fused_slab_forward_backward(q, k_buf, v_buf, grad_out, plan: SlabPlan, extent, ks, dl, ca, scale):
    """Forward and backward of one slab with already-assembled K/V buffers.
    Returns (out, lse, dq, dk_buf, dv_buf); the caller reduces the halo parts."""
    rank = len(extent)
    slab = _slab(plan, extent)
    one = (1,) * rank
    out, lse = _cuda.fused_forward(q, k_buf, v_buf, ks, one, dl, ca, scale, slab=slab)
    dq, dk, dv, _, _ = _cuda.fused_backward(q, k_buf, v_buf, out, lse, grad_out, None, ks, one, dl, ca, scale, slab=slab)
    return out, lse, dq, dk, dv


class _ShardedNA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, extent, ks, dl, ca, scale, plans, rank, group):
        k_buf, v_buf = exchange_halos([k, v], plans, rank, group)
        slab = _slab(plans[rank], extent)
        one = (1,) * len(extent)
        out, lse = _cuda.fused_forward(q, k_buf, v_buf, ks, one, dl, ca, scale, slab=slab)
        ctx.save_for_backward(q, k_buf, v_buf, out, lse)
        ctx.args = (extent, ks, dl, ca, scale, plans, rank, group, slab, one)
        return out, lse

    @staticmethod
    def backward(ctx, grad_out, grad_lse):
        q, k_buf, v_buf, out, lse = ctx.saved_tensors
        extent, ks, dl, ca, scale, plans, rank, group, slab, one = ctx.args
        if grad_out is None:
            grad_out = torch.zeros_like(out)
        dq, dk, dv, _, _ = _cuda.fused_backward(q, k_buf, v_buf, out, lse, grad_out, grad_lse, ks, one, dl, ca,
                                                scale, slab=slab)
        dk, dv = reduce_halo_grads_many([dk, dv], plans, rank, group)
        return (dq, dk, dv) + (None,) * 8


def na_sharded(query, key, value, global_extent: int, kernel_size, dilation=1, is_causal=False,
               scale: Optional[float] = None, return_lse: bool = False, group=None):
    """Neighborhood attention on a volume sharded along its leading spatial axis.

    Each rank passes its own planes of q/k/v (``[B, T_local, ..., H, D]``, the
    contiguous balanced split of ``global_extent`` planes, see ``shard_bounds``).
    Stride is 1.  Returns this rank's planes of the output (and LSE)."""
    rank_nd = query.dim() - 3
    tup = lambda x: tuple(x) if isinstance(x, (tuple, list)) else (x,) * rank_nd
    ks, dl, ca = tup(kernel_size), tup(dilation), tuple(bool(c) for c in tup(is_causal))
    world = dist.get_world_size(group)
    me = dist.get_rank(group)
    plans = all_plans(global_extent, world, ks[0], dl[0], ca[0])
    if query.shape[1] != plans[me].q_hi - plans[me].q_lo:
        raise ValueError(f"rank {me} must hold planes [{plans[me].q_lo}, {plans[me].q_hi}) of the leading axis")
    extent = (global_extent,) + tuple(query.shape[2:2 + rank_nd - 1])
    scale_value = query.shape[-1] ** -0.5 if scale is None else float(scale)
    out, lse = _ShardedNA.apply(query, key, value, extent, ks, dl, ca, scale_value, plans, me, group)
    return (out, lse) if return_lse else out
