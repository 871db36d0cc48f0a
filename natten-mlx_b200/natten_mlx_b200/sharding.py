"""Multi-GPU use of the path: batch/head shards need no communication; a large
volume can also be split along its leading spatial axis, with a K/V halo
exchange in the forward and the reverse dK/dV halo reduction in the backward.

The reference is single-device (it has no distributed code); this module is
what makes its operators span the GPUs of one box.  One process per GPU.  Two
transports move the halo planes: on GPUs under an NCCL group the library's own
copy kernel writes them straight into the consumer's K/V buffer over NVLink
(buffers in symmetric memory, ordered by the library's flag barrier; see
``PeerTransport``); otherwise ``torch.distributed`` point-to-point (gloo in the
CPU tests, NCCL send/recv when asked for).  Either way halo planes are in
local memory before any kernel reads them.

Window positions are evaluated in global coordinates: each rank passes its
slab offsets to the kernels (``Slab``), so results equal the unsharded call.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import ctypes
import warnings

import torch
import torch.distributed as dist

from . import _lib
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


def balance_by_tokens(sizes: Sequence[Sequence[int]], world: int) -> List[List[int]]:
    """Samples of a variable-size batch for each rank, balanced by token count (the product of a sample's
    extents) rather than by sample count: largest sample first onto the lightest rank.  Every rank gets at
    least one sample when there are enough; the lists hold sample indices in ascending order."""
    if world < 1:
        raise ValueError("world must be positive")
    tokens = []
    for i, s in enumerate(sizes):
        n = 1
        for x in (s if isinstance(s, (list, tuple)) else (s,)):
            n *= int(x)
        tokens.append((n, i))
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for n, i in sorted(tokens, key=lambda t: (-t[0], t[1])):
        r = min(range(world), key=lambda j: (load[j], len(out[j]), j))
        out[r].append(i)
        load[r] += n
    return [sorted(x) for x in out]


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


def halo_transfers(plans: Sequence[SlabPlan]) -> List[Tuple[int, int, int, int]]:
    """Every (owner, borrower, lo, hi): planes [lo, hi) owned by ``owner`` that ``borrower``'s queries address."""
    out = []
    for owner in plans:
        for other in plans:
            if other.rank == owner.rank:
                continue
            lo, hi = _overlap(owner.q_lo, owner.q_hi, other.kv_lo, other.kv_hi)
            if hi > lo:
                out.append((owner.rank, other.rank, lo, hi))
    return out


def staging_layout(plans: Sequence[SlabPlan]) -> Tuple[dict, int]:
    """Where an owner keeps the gradient partials it receives: {(owner, borrower): first plane of that borrower's
    range in the owner's staging area}, and the number of planes the largest staging area holds."""
    offsets, used = {}, [0] * len(plans)
    for owner, borrower, lo, hi in halo_transfers(plans):
        offsets[(owner, borrower)] = used[owner]
        used[owner] += hi - lo
    return offsets, max(used) if used else 0


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class _Lease:
    """One symmetric allocation handed out by a ``PeerTransport``; goes back to its pool on ``release`` (or when
    the last reference dies).

    ``read_epoch`` is the transport's barrier count when a kernel reading the allocation was last queued on this
    rank's stream (``mark_read``).  Another rank may write into the allocation once a barrier queued after that
    point has completed; ``needs_barrier`` tells whether such a barrier has been queued yet.  Every rank makes
    the same calls in the same order, so every rank reaches the same answer."""

    def __init__(self, transport, nbytes, tensor, ptrs, read_epoch=-1):
        self.transport, self.nbytes, self.tensor, self.ptrs = transport, nbytes, tensor, ptrs
        self.read_epoch = read_epoch
        self.persistent = False
        self.live = True

    def mark_read(self):
        self.read_epoch = self.transport.epoch

    def needs_barrier(self) -> bool:
        return self.transport.epoch <= self.read_epoch

    def release(self):
        if self.live:
            self.live = False
            for key in [k for k, v in _kv_registry.items() if v[0] is self]:
                del _kv_registry[key]
            self.transport._pool.setdefault(self.nbytes, []).append((self.tensor, self.ptrs, self.read_epoch))

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


_kv_registry = {}      # (data_ptr, shape) of a tensor handed out by peer_kv_buffers -> (lease, index)


class PeerTransport:
    """Halo transport of one process group over peer memory.

    Buffers come from ``torch.distributed._symmetric_memory`` (every rank's allocation is mapped into every other
    rank's address space); the data is moved by the library's copy kernel (``natten_b200_peer_copy2d``: plain
    16-byte stores into the consumer's memory) and ordered by its flag barrier (``natten_b200_peer_barrier``,
    bounded waits).  All ranks of the group must make the same sequence of calls, on one stream each; allocations
    are collective and are kept in a pool, so steady-state steps allocate nothing."""

    def __init__(self, group=None):
        import torch.distributed._symmetric_memory as symm
        self._symm = symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._pool = {}
        self.epoch = 0
        flags = symm.empty(64, dtype=torch.int32, device=self.device)
        flags.zero_()
        torch.cuda.synchronize(self.device)
        self._flags = flags
        self._flag_handle = symm.rendezvous(flags, self.group)
        self._flag_ptrs = (ctypes.c_uint64 * self.world)(*[int(p) for p in self._flag_handle.buffer_ptrs])
        dist.barrier(self.group)              # every rank's flag block is zero before anyone publishes into it

    def barrier(self):
        """Queue a barrier over the ranks on the current stream."""
        self.epoch += 1
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.load().natten_b200_peer_barrier(self._flag_ptrs, self.world, self.rank, self.epoch, 0,
                                                        ctypes.c_void_p(stream)))

    def acquire(self, nbytes: int) -> _Lease:
        """A symmetric allocation of ``nbytes`` (the same on every rank; collective when the pool has none)."""
        free = self._pool.get(nbytes)
        if free:
            tensor, ptrs, read_epoch = free.pop()
            return _Lease(self, nbytes, tensor, ptrs, read_epoch)
        tensor = self._symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        handle = self._symm.rendezvous(tensor, self.group)
        return _Lease(self, nbytes, tensor, [int(p) for p in handle.buffer_ptrs])

    def copy2d(self, dst_ptr, dst_pitch, src_ptr, src_pitch, width, rows, dma: bool = False):
        """Pitched copy on the current stream, by the library's copy kernel or (``dma``) by a copy engine."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        fn = _lib.load().natten_b200_peer_copy2d_dma if dma else _lib.load().natten_b200_peer_copy2d
        _lib.check(fn(ctypes.c_void_p(dst_ptr), dst_pitch, ctypes.c_void_p(src_ptr), src_pitch, width, rows,
                      ctypes.c_void_p(stream)))

    @property
    def side_stream(self):
        """A high-priority stream for exchanges that run under kernels of the current stream."""
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=self.device, priority=-1)
        return self._side


_transports = {}
_transport_refused = {}


def peer_transport(group=None) -> Optional[PeerTransport]:
    """The group's ``PeerTransport`` (created on first use, collectively), or None where symmetric memory cannot
    be set up (the reason is kept in a warning); callers then use point-to-point transfers."""
    key = group if group is not None else dist.group.WORLD
    if key in _transports:
        return _transports[key]
    if key in _transport_refused:
        return None
    try:
        _transports[key] = PeerTransport(group)
    except (RuntimeError, ImportError, AttributeError) as err:
        _transport_refused[key] = str(err)
        warnings.warn(f"peer-memory halo transport unavailable, using send/recv: {err}")
        return None
    return _transports[key]


def _use_peer(tensor: torch.Tensor, group, transport: str) -> bool:
    if transport == "p2p":
        return False
    ok = (tensor.is_cuda and dist.get_backend(group) == "nccl" and dist.get_world_size(group) > 1
          and _plane_bytes(tensor, 1) % 16 == 0 and tensor.data_ptr() % 16 == 0)
    if transport == "peer" and not ok:
        raise ValueError("the peer-memory transport needs CUDA tensors whose planes are multiples of 16 bytes and an "
                         "NCCL group of more than one rank")
    if not ok:
        return False
    t = peer_transport(group)
    if t is None and transport == "peer":
        raise RuntimeError(f"peer-memory transport unavailable: {_transport_refused.get(group if group is not None else dist.group.WORLD)}")
    return t is not None


def _plane_bytes(t: torch.Tensor, axis: int) -> int:
    n = t.element_size()
    for x in t.shape[axis + 1:]:
        n *= x
    return n


def _kv_layout(shapes_dtypes, plans, axis):
    """Byte offset of every tensor's buffer inside one allocation, and the allocation's size: each buffer has room
    for the widest [kv_lo, kv_hi) range of any rank, so that the layout is the same on every rank."""
    span = max(p.kv_hi - p.kv_lo for p in plans)
    offs, total = [], 0
    for shape, dtype in shapes_dtypes:
        n = torch.empty((), dtype=dtype).element_size() * span
        for i, x in enumerate(shape):
            if i != axis:
                n *= x
        offs.append(total)
        total += _align(n)
    return offs, total


def _buffer_view(lease, off, local_shape, dtype, me, axis):
    shape = list(local_shape)
    shape[axis] = me.kv_hi - me.kv_lo
    n = torch.empty((), dtype=dtype).element_size()
    for x in shape:
        n *= x
    return lease.tensor[off: off + n].view(dtype).view(shape)


def peer_kv_buffers(local_shape, dtype, plans: Sequence[SlabPlan], rank: int, count: int = 2, group=None, axis: int = 1):
    """``count`` tensors of ``local_shape`` (K, V, ...) for this rank's planes that live inside one symmetric
    allocation, each with room for its halo planes around it: (tensors, lease).  A caller that produces its K/V
    into them saves ``na_sharded`` the copy of the owned planes into a halo buffer (the neighbours' planes are
    written around them in place).  Collective.  ``lease.release()`` gives the memory back."""
    t = peer_transport(group)
    if t is None:
        raise RuntimeError("peer-memory transport unavailable")
    me = plans[rank]
    offs, total = _kv_layout([(local_shape, dtype)] * count, plans, axis)
    lease = t.acquire(total)
    lease.persistent = True
    out = []
    for i in range(count):
        own = _buffer_view(lease, offs[i], local_shape, dtype, me, axis).narrow(axis, me.q_lo - me.kv_lo, me.q_hi - me.q_lo)
        _kv_registry[(own.data_ptr(), tuple(own.shape))] = (lease, i)
        out.append(own)
    return out, lease


def _registered(locals_):
    """The lease whose buffers ``locals_`` are, in order (see ``peer_kv_buffers``), or None."""
    lease = None
    for i, x in enumerate(locals_):
        hit = _kv_registry.get((x.data_ptr(), tuple(x.shape)))
        if hit is None or hit[1] != i or (lease is not None and hit[0] is not lease):
            return None
        lease = hit[0]
    return lease


def exchange_halos_peer(locals_: Sequence[torch.Tensor], plans: Sequence[SlabPlan], rank: int, group=None,
                        axis: int = 1, aside: bool = False):
    """``exchange_halos`` over peer memory: (buffers, lease).  Every rank writes the planes its neighbours need
    straight into their buffers, then a barrier tells everyone that its planes have arrived (a barrier before
    the writes is only queued when none has been queued since the buffers were last read).  The buffers are
    views of the lease's allocation; the caller calls ``lease.mark_read()`` after queueing the kernels that read
    them and, unless the lease is persistent, ``lease.release()`` when nothing reads them any more.

    ``aside``: the barriers and the writes (then by copy engines) are queued on the transport's side stream, which
    first waits for the current stream; the result gains a third element, the event after which the halo planes
    are there.  Kernels that read only owned planes can then run on the current stream in the meantime."""
    t = peer_transport(group)
    me = plans[rank]
    rows = 1
    for x in locals_[0].shape[:axis]:
        rows *= x
    pb = [_plane_bytes(x, axis) for x in locals_]
    offs, total = _kv_layout([(x.shape, x.dtype) for x in locals_], plans, axis)
    lease = _registered(locals_)
    if lease is None:
        lease = t.acquire(total)
        locals_ = [x if x.is_contiguous() else x.contiguous() for x in locals_]
        pitch = [(me.q_hi - me.q_lo) * b for b in pb]
    else:
        pitch = [(me.kv_hi - me.kv_lo) * b for b in pb]       # the owned planes already sit inside the buffers
    transfers = [x for x in halo_transfers(plans) if x[0] == rank]
    bufs = [_buffer_view(lease, offs[i], local.shape, local.dtype, me, axis) for i, local in enumerate(locals_)]

    def own_planes():
        if not lease.persistent:
            for buf, local in zip(bufs, locals_):
                buf.narrow(axis, me.q_lo - me.kv_lo, me.q_hi - me.q_lo).copy_(local)

    def exchange(dma):
        if lease.needs_barrier():
            t.barrier()                           # nobody still reads the buffers the writes below go to
        for i, local in enumerate(locals_):       # what the neighbours wait for goes first
            for _, borrower, lo, hi in transfers:
                other = plans[borrower]
                t.copy2d(lease.ptrs[borrower] + offs[i] + (lo - other.kv_lo) * pb[i], (other.kv_hi - other.kv_lo) * pb[i],
                         local.data_ptr() + (lo - me.q_lo) * pb[i], pitch[i], (hi - lo) * pb[i], rows, dma=dma)

    if not aside:
        exchange(False)
        own_planes()
        t.barrier()                               # the planes others wrote into this rank's buffers have arrived
        return bufs, lease
    main = torch.cuda.current_stream(t.device)
    side = t.side_stream
    side.wait_stream(main)                        # the K/V to lend exist; earlier readers of the buffers are done
    with torch.cuda.stream(side):
        exchange(True)
        t.barrier()
        arrived = torch.cuda.Event()
        arrived.record(side)
    for x in locals_:
        x.record_stream(side)
    own_planes()
    return bufs, lease, arrived


class _PeerReduce:
    """The halo reduction of dK / dV over peer memory, in its two halves: ``open`` reserves the staging areas (and
    queues the barrier that protects them, if one is due) and knows where this rank's partial sums go;
    ``close`` queues the arrival barrier and adds what the neighbours delivered into the owned planes.  Between
    the two the partial sums are delivered either by the copy kernel (``push``) or by the dK/dV kernel itself
    (``halo_out``: its epilogue stores the halo planes' gradients straight into the owner's staging area)."""

    def __init__(self, like: Sequence[torch.Tensor], plans, rank, group, axis=1):
        self.t = peer_transport(group)
        self.plans, self.rank, self.axis = plans, rank, axis
        self.me = plans[rank]
        self.rows = 1
        for x in like[0].shape[:axis]:
            self.rows *= x
        self.pb = [_plane_bytes(x, axis) for x in like]
        self.where, span = staging_layout(plans)
        self.offs, total = [], 0
        for b in self.pb:
            self.offs.append(total)
            total += _align(self.rows * span * b)
        self.transfers = halo_transfers(plans)
        self.lease = None
        if total:
            self.lease = self.t.acquire(total)
            if self.lease.needs_barrier():
                self.t.barrier()                  # the owners have finished with what the last call left there

    def target(self, i: int, owner: int) -> int:
        """Address, in this process, of the area where ``owner`` keeps this rank's partial sums of tensor ``i``."""
        return self.lease.ptrs[owner] + self.offs[i] + self.where[(owner, self.rank)] * self.rows * self.pb[i]

    def halo_out(self):
        """(planes_below, planes_above, dk_below, dv_below, dk_above, dv_above) for the dK/dV kernel, or None when
        the halo planes of this rank do not belong to its two direct neighbours alone."""
        me, below, above = self.me, self.me.q_lo - self.me.kv_lo, self.me.kv_hi - self.me.q_hi
        mine = [(o, lo, hi) for o, b, lo, hi in self.transfers if b == self.rank]
        want = ([(self.rank - 1, me.kv_lo, me.q_lo)] if below else []) + ([(self.rank + 1, me.q_hi, me.kv_hi)] if above else [])
        if sorted(mine) != sorted(want) or len(self.pb) != 2:
            return None
        lo = [self.target(i, self.rank - 1) if below else 0 for i in range(2)]
        hi = [self.target(i, self.rank + 1) if above else 0 for i in range(2)]
        return (below, above, lo[0], lo[1], hi[0], hi[1])

    def push(self, grad_bufs):
        """Deliver the partial sums held in the halo planes of ``grad_bufs`` with the copy kernel."""
        me = self.me
        for i, g in enumerate(grad_bufs):
            for owner, borrower, lo, hi in self.transfers:
                if borrower != self.rank:
                    continue
                # the owner's area holds rows of (hi - lo) planes for this borrower, densely: pitch = width
                self.t.copy2d(self.target(i, owner), (hi - lo) * self.pb[i], g.data_ptr() + (lo - me.kv_lo) * self.pb[i],
                              (me.kv_hi - me.kv_lo) * self.pb[i], (hi - lo) * self.pb[i], self.rows)

    def close(self, grad_bufs) -> List[torch.Tensor]:
        me, axis = self.me, self.axis
        owns = [g.narrow(axis, me.q_lo - me.kv_lo, me.q_hi - me.q_lo) for g in grad_bufs]
        if self.lease is None:
            return owns
        self.t.barrier()                          # the partials for this rank's planes have arrived
        for i, own in enumerate(owns):
            for owner, borrower, lo, hi in self.transfers:
                if owner != self.rank:
                    continue
                shape = list(own.shape)
                shape[axis] = hi - lo
                n = 1
                for x in shape:
                    n *= x
                start = self.offs[i] + self.where[(owner, borrower)] * self.rows * self.pb[i]
                piece = self.lease.tensor[start: start + n * own.element_size()].view(own.dtype).view(shape)
                own.narrow(axis, lo - me.q_lo, hi - lo).add_(piece)
        self.lease.mark_read()
        self.lease.release()
        self.lease = None
        return owns


def reduce_halo_grads_peer(grad_bufs: Sequence[torch.Tensor], plans: Sequence[SlabPlan], rank: int, group=None,
                           axis: int = 1) -> List[torch.Tensor]:
    """``reduce_halo_grads_many`` over peer memory: partial sums are written into the owner's staging area by the
    copy kernel, the owner adds them into its planes."""
    red = _PeerReduce(grad_bufs, plans, rank, group, axis)
    if red.lease is not None:
        red.push(grad_bufs)
    return red.close(grad_bufs)


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


def slab_forward_planes(q, k_buf, v_buf, out, lse, plan: SlabPlan, extent, ks, dl, ca, scale, p0: int, p1: int):
    """The fused forward of the local query planes [p0, p1) of a slab, written into those planes of ``out`` and
    ``lse``.  A range of planes of several samples is not dense in memory, so it is launched sample by sample."""
    if p1 <= p0:
        return
    rank = len(extent)
    part = _cuda.Slab(tuple(extent), (plan.q_lo + p0,) + (0,) * (rank - 1), (plan.kv_lo,) + (0,) * (rank - 1))
    one = (1,) * rank
    for b in range(q.shape[0]):
        _cuda.fused_forward(q[b:b + 1, p0:p1], k_buf[b:b + 1], v_buf[b:b + 1], ks, one, dl, ca, scale, slab=part,
                            out=out[b:b + 1, p0:p1], lse=lse[b:b + 1, p0:p1])


def _tensor_core_slab(q, k_buf, ks, one, dl, ca, scale, slab) -> bool:
    """Whether the fused backward of this slab runs on the tensor-core kernels (which can deliver halo gradients)."""
    if q.dtype not in (torch.float16, torch.bfloat16) or _cuda.get_fused_path() == "simt":
        return False
    geom = _cuda._geom(q, k_buf, q.dim() - 3, ks, one, dl, ca, _cuda._scale(scale, q.shape[-1]), slab=slab)
    try:
        return "unsupported" not in _lib.describe_plan(geom)
    except ValueError:
        return False


class _ShardedNA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, extent, ks, dl, ca, scale, plans, rank, group, transport):
        peer = _use_peer(q, group, transport)
        lease = None
        me = plans[rank]
        slab = _slab(me, extent)
        one = (1,) * len(extent)
        below, above = me.q_lo - me.kv_lo, me.kv_hi - me.q_hi
        planes = me.q_hi - me.q_lo
        if peer and below + above > 0 and planes > below + above and q.shape[0] <= 8:
            # The planes whose windows stay inside this rank's own planes are computed while the halo planes
            # travel (copy engines and barriers on a second stream); the boundary planes follow.  A slab of
            # several samples is not dense in memory, so the pieces are launched sample by sample.
            (k_buf, v_buf), lease, arrived = exchange_halos_peer([k, v], plans, rank, group, aside=True)
            q = q if q.is_contiguous() else q.contiguous()
            out = torch.empty_like(q)
            lse = torch.empty(q.shape[:-1], dtype=torch.float32, device=q.device)
            args = (q, k_buf, v_buf, out, lse, me, extent, ks, dl, ca, scale)
            slab_forward_planes(*args, below, planes - above)
            torch.cuda.current_stream(q.device).wait_event(arrived)
            slab_forward_planes(*args, 0, below)
            slab_forward_planes(*args, planes - above, planes)
        else:
            if peer:
                (k_buf, v_buf), lease = exchange_halos_peer([k, v], plans, rank, group)
            else:
                k_buf, v_buf = exchange_halos([k, v], plans, rank, group)
            out, lse = _cuda.fused_forward(q, k_buf, v_buf, ks, one, dl, ca, scale, slab=slab)
        if lease is not None:
            lease.mark_read()
            if not lease.persistent and not any(ctx.needs_input_grad[:3]):
                lease.release()               # nothing is saved for a backward
                lease = None
        ctx.save_for_backward(q, k_buf, v_buf, out, lse)
        ctx.lease = lease
        ctx.args = (extent, ks, dl, ca, scale, plans, rank, group, slab, one, peer)
        return out, lse

    @staticmethod
    def backward(ctx, grad_out, grad_lse):
        q, k_buf, v_buf, out, lse = ctx.saved_tensors
        extent, ks, dl, ca, scale, plans, rank, group, slab, one, peer = ctx.args
        if grad_out is None:
            grad_out = torch.zeros_like(out)
        red = halo = None
        if peer:
            # staging areas first: with the tensor-core kernels the dK/dV kernel itself delivers the halo planes'
            # partial sums into the owners' staging areas while it computes
            red = _PeerReduce([k_buf, v_buf], plans, rank, group)
            if red.lease is not None and _tensor_core_slab(q, k_buf, ks, one, dl, ca, scale, slab):
                halo = red.halo_out()
        dq, dk, dv, _, _ = _cuda.fused_backward(q, k_buf, v_buf, out, lse, grad_out, grad_lse, ks, one, dl, ca,
                                                scale, slab=slab, halo_out=halo)
        if ctx.lease is not None:
            ctx.lease.mark_read()
            if not ctx.lease.persistent:
                ctx.lease.release()
            ctx.lease = None
        if peer:
            if halo is None and red.lease is not None:
                red.push([dk, dv])
            dk, dv = red.close([dk, dv])
        else:
            dk, dv = reduce_halo_grads_many([dk, dv], plans, rank, group)
        return (dq, dk, dv) + (None,) * 9


def na_sharded(query, key, value, global_extent: int, kernel_size, dilation=1, is_causal=False,
               scale: Optional[float] = None, return_lse: bool = False, group=None, transport: str = "auto"):
    """Neighborhood attention on a volume sharded along its leading spatial axis.

    Each rank passes its own planes of q/k/v (``[B, T_local, ..., H, D]``, the
    contiguous balanced split of ``global_extent`` planes, see ``shard_bounds``).
    Stride is 1.  ``transport``: "peer" (the library's copy kernel over peer memory), "p2p" (point-to-point
    send/recv of the group's backend) or "auto" (peer on GPUs under NCCL, else p2p).  Returns this rank's planes
    of the output (and LSE)."""
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
    if transport not in ("auto", "peer", "p2p"):
        raise ValueError(f"transport must be 'auto', 'peer' or 'p2p', got {transport!r}")
    out, lse = _ShardedNA.apply(query, key, value, extent, ks, dl, ca, scale_value, plans, me, group, transport)
    return (out, lse) if return_lse else out
