"""Host-resident tensors: fused forward + backward streamed through the GPU.

The operators of this package take device tensors.  A caller whose q/k/v and
output cotangent live in (pinned) host memory — the situation of the
reference's users, whose arrays sit in unified memory — would otherwise copy
everything in, compute, and copy everything out, one after the other.  Neighbourhood
attention is independent across the batch axis (`src/natten_mlx/_core/pure.py:242-248`
reduces over the neighbourhood and the head dimension only), so
:class:`HostPipeline` cuts the batch into slabs and keeps three streams busy:
slab ``i + 1`` travels host→device while slab ``i`` is computed and the results
of slab ``i - 1`` travel device→host.  The two copy directions use separate
copy engines, so the call approaches the time of the slower direction instead of
the sum of all three phases.

Results are bit-identical to one call over the whole batch: slabs are whole
samples, and no kernel of the package reduces across samples.
"""

from __future__ import annotations

from typing import Sequence

import torch

from . import _lib
from ._core import cuda as backend
from .utils.params import normalize_kernel_size, normalize_tuple_param


_STREAMS = {}


class HostPipeline:
    """Reusable plan for ``fused forward + backward`` on host tensors of one geometry.

    ``shape`` is the q layout ``[B, spatial..., heads_q, D]``; ``heads_kv`` defaults to
    ``heads_q``.  Input and result buffers for two slabs, the scratch of the backward and the geometry of a
    slab are set up once; a run only queues copies and the two library calls per slab.
    """

    def __init__(self, shape: Sequence[int], dtype: torch.dtype, device, kernel_size, dilation=1, is_causal=False,
                 stride=1, scale=None, heads_kv=None, slabs: int = 4):
        shape = tuple(int(s) for s in shape)
        rank = len(shape) - 3
        if rank not in (1, 2, 3):
            raise ValueError("HostPipeline: shape must be [B, spatial..., heads, D] with 1 to 3 spatial axes")
        self.rank = rank
        self.shape = shape
        self.kv_shape = shape[:-2] + (int(heads_kv or shape[-2]), shape[-1])
        self.dtype = dtype
        self.device = torch.device(device)
        self.kernel_size = normalize_kernel_size(kernel_size, rank)
        self.dilation = tuple(int(x) for x in normalize_tuple_param(dilation, rank, "dilation"))
        self.stride = tuple(int(x) for x in normalize_tuple_param(stride, rank, "stride"))
        self.is_causal = tuple(bool(c) for c in normalize_tuple_param(is_causal, rank, "is_causal"))
        self.scale = scale
        batch = shape[0]
        slabs = max(1, min(int(slabs), batch))
        step = -(-batch // slabs)
        self.ranges = [(b0, min(batch, b0 + step)) for b0 in range(0, batch, step)]
        per = max(b1 - b0 for b0, b1 in self.ranges)
        mk = lambda s, dt=dtype: torch.empty((per,) + tuple(s[1:]), dtype=dt, device=self.device)
        # two sets of device buffers: the staged inputs q, k, v, cotangent and the results out, lse, dq, dk, dv.
        # Everything a slab needs on the device exists before the first run: a run allocates nothing and builds
        # no geometry (the host work per slab is what limits how finely the batch can be cut).
        out_shape = (shape[0],) + backend._out_shape(shape[1:1 + rank], self.stride) + tuple(shape[-2:])
        self.stage = [[mk(shape), mk(self.kv_shape), mk(self.kv_shape), mk(out_shape)] for _ in range(2)]
        self.result = [[mk(out_shape), mk(out_shape[:-1], torch.float32), mk(shape), mk(self.kv_shape), mk(self.kv_shape)]
                       for _ in range(2)]
        self._calls = {}          # samples in a slab -> (geometry, scratch bytes)
        self._scratch = [None, None]
        # the three streams are shared by every plan of a device, so that consecutive runs of different
        # plans keep streaming (the copy-in of the next run starts under the tail of the previous one)
        key = (self.device.type, self.device.index if self.device.index is not None else torch.cuda.current_device())
        if key not in _STREAMS:
            _STREAMS[key] = tuple(torch.cuda.Stream(device=self.device) for _ in range(3))
        self.s_in, self.s_cmp, self.s_out = _STREAMS[key]
        self._free = [None, None]      # event: the compute stream has finished with the staged inputs of set b
        self._drained = [None, None]   # event: the results of set b have left for the host

    def _call(self, n: int, b: int):
        """Geometry and scratch of a slab of ``n`` samples on buffer set ``b`` (built once)."""
        hit = self._calls.get(n)
        if hit is None:
            q, k = self.stage[0][0][:n], self.stage[0][1][:n]
            geom = backend._geom(q, k, self.rank, self.kernel_size, self.stride, self.dilation, self.is_causal,
                                 backend._scale(self.scale, self.shape[-1]))
            nbytes = int(_lib.load().natten_b200_fused_backward_scratch_bytes(geom))
            hit = self._calls[n] = (geom, nbytes)
        if self._scratch[b] is None or self._scratch[b].numel() < max(hit[1], 16):
            self._scratch[b] = torch.empty(max(hit[1], 16), dtype=torch.uint8, device=self.device)
        return hit

    def run(self, q, k, v, dout, out, dq, dk, dv, wait: bool = True):
        """All arguments are host tensors (pinned for overlap); the last four are written.

        With ``wait=False`` the current stream is not made to wait for the results: call
        :meth:`join` (of the last plan run) before reading them.  Several runs may be queued."""
        if tuple(q.shape) != self.shape or tuple(k.shape) != self.kv_shape or tuple(v.shape) != self.kv_shape:
            raise ValueError("HostPipeline.run: tensor shapes do not match the plan")
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_cmp, self.s_out):      # work already queued on the current stream comes first
            s.wait_stream(cur)
        lib = _lib.load()
        free, drained = self._free, self._drained
        p = lambda t: t.data_ptr()
        for i, (b0, b1) in enumerate(self.ranges):
            n = b1 - b0
            b = i % 2
            st, rs = self.stage[b], self.result[b]
            with torch.cuda.stream(self.s_in):
                if free[b] is not None:
                    self.s_in.wait_event(free[b])
                for d, h in zip(st, (q, k, v, dout)):
                    d[:n].copy_(h[b0:b1], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            geom, nbytes = self._call(n, b)
            with torch.cuda.stream(self.s_cmp), torch.cuda.device(self.device):
                self.s_cmp.wait_event(ready)
                if drained[b] is not None:
                    self.s_cmp.wait_event(drained[b])      # the results of the slab before last have been read
                stream = self.s_cmp.cuda_stream
                _lib.check(lib.natten_b200_fused_forward(geom, p(st[0]), p(st[1]), p(st[2]), None, None, p(rs[0]), p(rs[1]),
                                                         stream))
                _lib.check(lib.natten_b200_fused_backward(
                    geom, p(st[0]), p(st[1]), p(st[2]), None, None, p(rs[0]), p(rs[1]), p(st[3]), None, p(rs[2]), p(rs[3]),
                    p(rs[4]), None, None, p(self._scratch[b]), nbytes, stream))
                done = torch.cuda.Event()
                done.record(self.s_cmp)
                free[b] = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for h, d in zip((out, dq, dk, dv), (rs[0], rs[2], rs[3], rs[4])):
                    h[b0:b1].copy_(d[:n], non_blocking=True)
                gone = torch.cuda.Event()
                gone.record(self.s_out)
                drained[b] = gone
        if wait:
            self.join()

    def join(self):
        """Make the current stream wait for everything queued on the pipeline's streams."""
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self.s_cmp)
        cur.wait_stream(self.s_out)
