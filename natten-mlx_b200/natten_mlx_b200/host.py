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

from ._core import cuda as backend
from .utils.params import normalize_kernel_size, normalize_tuple_param


_STREAMS = {}


class HostPipeline:
    """Reusable plan for ``fused forward + backward`` on host tensors of one geometry.

    ``shape`` is the q layout ``[B, spatial..., heads_q, D]``; ``heads_kv`` defaults to
    ``heads_q``.  Staging buffers for two slabs are allocated once.
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
        mk = lambda s: torch.empty((per,) + tuple(s[1:]), dtype=dtype, device=self.device)
        # two sets of device staging buffers: q, k, v, cotangent
        self.stage = [[mk(shape), mk(self.kv_shape), mk(self.kv_shape), mk(shape)] for _ in range(2)]
        # the three streams are shared by every plan of a device, so that consecutive runs of different
        # plans keep streaming (the copy-in of the next run starts under the tail of the previous one)
        key = (self.device.type, self.device.index if self.device.index is not None else torch.cuda.current_device())
        if key not in _STREAMS:
            _STREAMS[key] = tuple(torch.cuda.Stream(device=self.device) for _ in range(3))
        self.s_in, self.s_cmp, self.s_out = _STREAMS[key]
        self._free = [None, None]    # event: the compute stream has finished with staging set b

    def run(self, q, k, v, dout, out, dq, dk, dv, wait: bool = True):
        """All arguments are host tensors (pinned for overlap); the last four are written.

        With ``wait=False`` the current stream is not made to wait for the results: call
        :meth:`join` (of the last plan run) before reading them.  Several runs may be queued."""
        if tuple(q.shape) != self.shape or tuple(k.shape) != self.kv_shape or tuple(v.shape) != self.kv_shape:
            raise ValueError("HostPipeline.run: tensor shapes do not match the plan")
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_cmp, self.s_out):      # work already queued on the current stream comes first
            s.wait_stream(cur)
        free = self._free
        for i, (b0, b1) in enumerate(self.ranges):
            n = b1 - b0
            st = self.stage[i % 2]
            with torch.cuda.stream(self.s_in):
                if free[i % 2] is not None:
                    self.s_in.wait_event(free[i % 2])
                for d, h in zip(st, (q, k, v, dout)):
                    d[:n].copy_(h[b0:b1], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(ready)
                qd, kd, vd, cd = (t[:n] for t in st)
                o, lse = backend.fused_forward(qd, kd, vd, self.kernel_size, self.stride, self.dilation, self.is_causal,
                                               self.scale)
                gq, gk, gv, _, _ = backend.fused_backward(qd, kd, vd, o, lse, cd, None, self.kernel_size, self.stride,
                                                          self.dilation, self.is_causal, self.scale)
                done = torch.cuda.Event()
                done.record(self.s_cmp)
                free[i % 2] = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for h, d in zip((out, dq, dk, dv), (o, gq, gk, gv)):
                    d.record_stream(self.s_out)
                    h[b0:b1].copy_(d, non_blocking=True)
        if wait:
            self.join()

    def join(self):
        """Make the current stream wait for everything queued on the pipeline's streams."""
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self.s_cmp)
        cur.wait_stream(self.s_out)
