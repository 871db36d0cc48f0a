"""CPU oracle for the neighborhood-attention hot path.

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU, the algorithm of the
reference's "pure" backend so that the CUDA kernels can be checked against it.
It is imported by the tests, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` and by nothing
else; the product package never imports it and has no CPU path of its own.

Integer index math is plain numpy; floating-point math is torch on the CPU
(float32 or float64) and gradients come from torch autograd of the restated
forward, which is what the reference does with ``mx.grad``
(src/natten_mlx/_core/pure.py:691-808).

Parity pin: the integer tables are checked against tables produced by the
reference's own ``utils/window.py`` and the float results against results of
the reference's own ``_core/pure.py`` / ``functional.py`` / ``merge.py`` /
``extras/allin1`` code executed over a torch-backed stand-in for the array
library it needs (the fixtures and their generator are in ``tests/golden``).

Every function names the reference lines it follows.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch


# ----------------------------------------------------------------------------
# integer window math
# ----------------------------------------------------------------------------

def window_start(p: int, length: int, ksize: int, dil: int) -> int:
    """First key index of a non-causal window (src/natten_mlx/utils/window.py:8-34)."""
    nh = ksize // 2
    if dil <= 1:
        s = max(p - nh, 0)
        if p + nh >= length:
            s += length - p - nh - 1
        return s
    if p - nh * dil < 0:
        return p % dil
    if p + nh * dil >= length:
        r = p % dil
        a = (length // dil) * dil
        b = length - a
        if r < b:
            return length - b + r - 2 * nh * dil
        return a + r - ksize * dil
    return p - nh * dil


def window_end(start: int, length: int, ksize: int, dil: int) -> int:
    """Half-open end of a non-causal window (src/natten_mlx/utils/window.py:37-39)."""
    return min(length, start + ksize * dil)


def pb_start(p: int, length: int, ksize: int, dil: int) -> int:
    """First relative-position-bias slot of a query (src/natten_mlx/utils/window.py:42-62)."""
    nh = ksize // 2
    if dil <= 1:
        v = nh
        if p < nh:
            v += nh - p
        if p + nh >= length:
            v += length - p - 1 - nh
        return v
    if p - nh * dil < 0:
        return ksize - 1 - (p // dil)
    if p + nh * dil >= length:
        return (length - p - 1) // dil
    return nh


def window_start_grouped(p: int, length: int, ksize: int, dil: int) -> int:
    """Dilation-group form of the window start
    (src/natten_mlx/extras/allin1/reference_impl.py:13-25)."""
    nh = ksize // 2
    g = p % dil
    i = p // dil
    lg = (length + dil - 1) // dil
    padded = lg * dil - length
    if g >= dil - padded:
        lg -= 1
    s = max(i - nh, 0)
    if i + nh >= lg:
        s += lg - i - nh - 1
    return s * dil + g


def query_positions(length: int, stride: int) -> np.ndarray:
    """Query coordinates on the stride lattice (src/natten_mlx/_core/pure.py:19-21)."""
    n = (length + stride - 1) // stride
    return (np.arange(n, dtype=np.int64) * stride).astype(np.int32)


def axis_table(qpos: np.ndarray, length: int, ksize: int, dil: int, causal: bool):
    """Per-axis neighbour index (clipped) and validity, shape [n_query, ksize]
    (src/natten_mlx/_core/pure.py:52-73)."""
    qpos = np.asarray(qpos, dtype=np.int64)
    steps = np.arange(ksize, dtype=np.int64)
    if causal == 2:  # whole axis (the dense route, src/natten_mlx/functional.py:141-187)
        raw = np.broadcast_to(steps[None, :], (len(qpos), ksize))
        return raw.astype(np.int32), np.ones_like(raw, dtype=bool)
    if causal:
        first = qpos - (ksize - 1) * dil
        raw = first[:, None] + steps[None, :] * dil
        ok = (raw >= 0) & (raw <= qpos[:, None]) & (raw < length)
    else:
        first = np.array([window_start(int(p), length, ksize, dil) for p in qpos], dtype=np.int64)
        last = np.array([window_end(int(s), length, ksize, dil) for s in first], dtype=np.int64)
        raw = first[:, None] + steps[None, :] * dil
        ok = (raw >= 0) & (raw < last[:, None])
    return np.clip(raw, 0, length - 1).astype(np.int32), ok


def neighbor_tables(extent: Sequence[int], ksize: Sequence[int], stride: Sequence[int],
                    dil: Sequence[int], causal: Sequence[bool]):
    """Linear neighbour index and validity for every query, any rank.

    Returns (lin [n_out..., K_vol] int64, valid [n_out..., K_vol] bool, out_shape).
    Slot order is row-major over the per-axis slots
    (src/natten_mlx/_core/pure.py:24-49, 76-106, 109-152).
    """
    rank = len(extent)
    idx, ok, outs = [], [], []
    for a in range(rank):
        qp = query_positions(extent[a], stride[a])
        i, v = axis_table(qp, extent[a], ksize[a], dil[a], int(causal[a]))
        idx.append(i.astype(np.int64))
        ok.append(v)
        outs.append(len(qp))
    lin = np.zeros([1] * (2 * rank), dtype=np.int64)
    valid = np.ones([1] * (2 * rank), dtype=bool)
    for a in range(rank):
        shape = [1] * (2 * rank)
        shape[a] = outs[a]
        shape[rank + a] = ksize[a]
        lin = lin * extent[a] + idx[a].reshape(shape)
        valid = valid & ok[a].reshape(shape)
    kvol = int(np.prod(ksize))
    lin = np.broadcast_to(lin, outs + list(ksize)).reshape(outs + [kvol])
    valid = np.broadcast_to(valid, outs + list(ksize)).reshape(outs + [kvol])
    return lin, valid, tuple(outs)


# ----------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------

def _tup(x, rank):
    if isinstance(x, (tuple, list)):
        assert len(x) == rank
        return tuple(x)
    return tuple(x for _ in range(rank))


def repeat_kv(x: torch.Tensor, rep: int) -> torch.Tensor:
    """GQA/MQA head expansion, consecutive repeats (src/natten_mlx/functional.py:29-33)."""
    return x if rep == 1 else torch.repeat_interleave(x, rep, dim=-2)


def _select_queries(q: torch.Tensor, extent, stride):
    for a in range(len(extent)):
        if stride[a] != 1:
            pos = torch.from_numpy(query_positions(extent[a], stride[a]).astype(np.int64))
            q = q.index_select(1 + a, pos)
    return q


def _gather(x: torch.Tensor, lin: np.ndarray, outs, kvol):
    """x [B, spatial..., H, D] -> neighbours [B, out..., H, K_vol, D]."""
    b, h, d = x.shape[0], x.shape[-2], x.shape[-1]
    flat = x.reshape(b, -1, h, d)
    g = flat.index_select(1, torch.from_numpy(np.ascontiguousarray(lin).reshape(-1).copy()))
    g = g.reshape(b, *outs, kvol, h, d)
    return g.movedim(-3, -2)


# ----------------------------------------------------------------------------
# split and fused operators (heads-last layout)
# ----------------------------------------------------------------------------

def na_qk(q, k, kernel_size, stride=1, dilation=1, is_causal=False, scale=None):
    """Masked logits [B, out..., H, K_vol]; invalid slots are -inf
    (src/natten_mlx/_core/pure.py:258-283, 320-359, 404-449)."""
    rank = q.dim() - 3
    ks, st, dl, ca = _tup(kernel_size, rank), _tup(stride, rank), _tup(dilation, rank), _tup(is_causal, rank)
    extent = tuple(q.shape[1:1 + rank])
    k = repeat_kv(k, q.shape[-2] // k.shape[-2])
    sc = q.shape[-1] ** -0.5 if scale is None else float(scale)
    lin, valid, outs = neighbor_tables(extent, ks, st, dl, ca)
    kvol = lin.shape[-1]
    kn = _gather(k, lin, outs, kvol)
    qs = _select_queries(q, extent, st)
    logits = (qs.unsqueeze(-2) * kn).sum(-1) * sc
    mask = torch.from_numpy(valid.copy()).reshape(1, *outs, 1, kvol)
    return torch.where(mask, logits, torch.full_like(logits, float("-inf")))


def na_av(attn, v, kernel_size, stride=1, dilation=1, is_causal=False):
    """Weighted sum of neighbour values, invalid slots weigh zero
    (src/natten_mlx/_core/pure.py:286-317, 362-401, 452-494)."""
    rank = v.dim() - 3
    ks, st, dl, ca = _tup(kernel_size, rank), _tup(stride, rank), _tup(dilation, rank), _tup(is_causal, rank)
    extent = tuple(v.shape[1:1 + rank])
    v = repeat_kv(v, attn.shape[-2] // v.shape[-2])
    lin, valid, outs = neighbor_tables(extent, ks, st, dl, ca)
    kvol = lin.shape[-1]
    if attn.shape[-1] != kvol:
        raise ValueError("attn neighborhood dimension must equal the kernel volume")
    if tuple(attn.shape[1:1 + rank]) != outs:
        raise ValueError("attn spatial dimensions must match ceil(input/stride)")
    vn = _gather(v, lin, outs, kvol)
    mask = torch.from_numpy(valid.copy()).reshape(1, *outs, 1, kvol)
    w = torch.where(mask, attn, torch.zeros_like(attn))
    return (w.unsqueeze(-1) * vn).sum(-2)


def full_attn_with_lse(q, k_extra, v_extra, scale):
    """Dense attention of every query over N_extra tokens, with log-sum-exp
    (src/natten_mlx/functional.py:71-104).  k_extra/v_extra: [B, N, H, D]."""
    b, h, d = q.shape[0], q.shape[-2], q.shape[-1]
    spatial = q.shape[1:-2]
    qf = q.reshape(b, -1, h, d).transpose(1, 2)
    kf = k_extra.transpose(1, 2)
    vf = v_extra.transpose(1, 2)
    logits = (qf @ kf.transpose(-1, -2)) * scale
    lse = torch.logsumexp(logits, dim=-1)
    out = torch.softmax(logits, dim=-1) @ vf
    out = out.transpose(1, 2).reshape(b, *spatial, h, d)
    lse = lse.transpose(1, 2).reshape(b, *spatial, h)
    return out, lse


def merge_attentions(outputs, lses):
    """Merge attention results that share queries (src/natten_mlx/merge.py:20-68)."""
    if len(outputs) < 2:
        raise ValueError("merge_attentions expects at least two outputs.")
    if len(outputs) != len(lses):
        raise ValueError("Number of outputs and LSE tensors must match.")
    ref = outputs[0].shape
    for o, l in zip(outputs, lses):
        if o.shape != ref or l.shape != ref[:-1]:
            raise ValueError("merge_attentions: shape does not match output 0")
    ls = [l.unsqueeze(-1).float() for l in lses]
    os_ = [o.float() for o in outputs]
    out = os_[0] - torch.sigmoid(ls[1] - ls[0]) * (os_[0] - os_[1])
    lse = ls[0] - torch.nn.functional.logsigmoid(ls[0] - ls[1])
    for i in range(2, len(os_)):
        out = out - torch.sigmoid(ls[i] - lse) * (out - os_[i])
        lse = lse - torch.nn.functional.logsigmoid(lse - ls[i])
    return out.to(outputs[0].dtype), lse.squeeze(-1)


def na(q, k, v, kernel_size, stride=1, dilation=1, is_causal=False, scale=None,
       return_lse=False, additional_keys=None, additional_values=None):
    """Fused neighborhood attention as the public functional composes it
    (src/natten_mlx/functional.py:207-473; math src/natten_mlx/_core/pure.py:155-255).

    When the kernel covers the whole extent on every axis (stride 1, no causal
    axis) the reference switches to dense attention over all keys
    (functional.py:141-187); for even kernels that differs from the window
    formula, so the oracle switches too.
    """
    rank = q.dim() - 3
    ks, st, dl, ca = _tup(kernel_size, rank), _tup(stride, rank), _tup(dilation, rank), _tup(is_causal, rank)
    rep = q.shape[-2] // k.shape[-2]
    sc = q.shape[-1] ** -0.5 if scale is None else float(scale)
    extent_ = tuple(q.shape[1:1 + rank])
    if all(kk >= e for kk, e in zip(ks, extent_)) and all(s == 1 for s in st) and not any(ca):
        ca = (2,) * rank
    logits = na_qk(q, k, ks, st, dl, ca, sc)
    lse = torch.logsumexp(logits, dim=-1)
    attn = torch.softmax(logits, dim=-1)
    out = na_av(attn, v, ks, st, dl, ca)
    if additional_keys is not None:
        extent = tuple(q.shape[1:1 + rank])
        qs = _select_queries(q, extent, st)
        oe, le = full_attn_with_lse(qs, repeat_kv(additional_keys, rep),
                                    repeat_kv(additional_values, rep), sc)
        out, lse = merge_attentions([out, oe], [lse, le])
    return (out, lse) if return_lse else out


def na_varlen(q, k, v, sizes, kernel_size, dilation=1, scale=None,
              return_lse=False, additional_keys=None, additional_values=None):
    """Per-sample extents inside padded tensors; padding comes back as zeros
    (src/natten_mlx/_core/pure.py:497-688).  ``sizes`` is [B] (1-D) or [B, rank].
    GQA, extra tokens and LSE follow ``na`` per sample (the reference's varlen
    entry points do not take them; padded LSE entries are defined as 0)."""
    rank = q.dim() - 3
    sizes = np.asarray(sizes).reshape(q.shape[0], rank)
    sc = q.shape[-1] ** -0.5 if scale is None else float(scale)
    out = torch.zeros_like(q)
    lse = torch.zeros(q.shape[:-1], dtype=torch.float32 if q.dtype != torch.float64 else q.dtype)
    for b in range(q.shape[0]):
        sl = (slice(b, b + 1),) + tuple(slice(0, int(s)) for s in sizes[b])
        ak = None if additional_keys is None else additional_keys[b:b + 1]
        av = None if additional_values is None else additional_values[b:b + 1]
        o, l = na(q[sl], k[sl], v[sl], kernel_size, 1, dilation, False, sc,
                  return_lse=True, additional_keys=ak, additional_values=av)
        out[sl] = o
        lse[sl] = l.to(lse.dtype)
    return (out, lse) if return_lse else out


# ----------------------------------------------------------------------------
# extras.allin1: QK + relative position bias, AV  (non-causal, stride 1)
# ----------------------------------------------------------------------------

def qk_rpb(q, k, rpb, kernel_size: int, dilation: int = 1, scale: Optional[float] = None):
    """logits = (scale*q).k_nbr + rpb[h, pb+slot] per axis, -inf where invalid
    (src/natten_mlx/extras/allin1/__init__.py:40-79, 112-150;
    src/natten_mlx/extras/allin1/functional.py:57-165, 260-318)."""
    rank = q.dim() - 3
    ks = int(kernel_size)
    dl = int(dilation)
    extent = tuple(q.shape[1:1 + rank])
    heads = q.shape[-2]
    logits = na_qk(q, k, (ks,) * rank, 1, (dl,) * rank, False, 1.0 if scale is None else float(scale))
    if rpb is None:
        return logits
    pb = [np.array([pb_start(p, extent[a], ks, dl) for p in range(extent[a])], dtype=np.int64)
          for a in range(rank)]
    steps = np.arange(ks, dtype=np.int64)
    if rank == 1:
        idx = torch.from_numpy(pb[0][:, None] + steps[None, :])            # [L, K]
        bias = rpb[:, idx]                                                 # [H, L, K]
        bias = bias.permute(1, 0, 2).unsqueeze(0)                          # [1, L, H, K]
    else:
        ih = torch.from_numpy(pb[0][:, None] + steps[None, :])            # [Hh, K]
        iw = torch.from_numpy(pb[1][:, None] + steps[None, :])            # [Ww, K]
        bias = rpb[:, ih[:, None, :, None], iw[None, :, None, :]]          # [H, Hh, Ww, K, K]
        bias = bias.reshape(heads, extent[0], extent[1], ks * ks).permute(1, 2, 0, 3).unsqueeze(0)
    return logits + bias.to(logits.dtype)


def av_fused(attn, v, kernel_size: int, dilation: int = 1):
    """(src/natten_mlx/extras/allin1/__init__.py:82-109, 153-180;
    src/natten_mlx/extras/allin1/functional.py:168-257, 321-368)."""
    rank = v.dim() - 3
    return na_av(attn, v, (int(kernel_size),) * rank, 1, (int(dilation),) * rank, False)


# ----------------------------------------------------------------------------
# gradients (autograd of the restated forward, src/natten_mlx/_core/pure.py:691-808)
# ----------------------------------------------------------------------------

def grads(fn, inputs, cotangents):
    """Run ``fn(*inputs)`` and return (outputs, grads wrt every tensor input).

    ``cotangents`` matches fn's outputs (a tensor or a tuple)."""
    leaves = [x.detach().clone().requires_grad_(True) if torch.is_tensor(x) and x.is_floating_point()
              else x for x in inputs]
    outs = fn(*leaves)
    outs_t = outs if isinstance(outs, tuple) else (outs,)
    cots = cotangents if isinstance(cotangents, (tuple, list)) else (cotangents,)
    loss = sum((o * c.to(o.dtype)).sum() for o, c in zip(outs_t, cots))
    wrt = [x for x in leaves if torch.is_tensor(x) and x.requires_grad]
    g = torch.autograd.grad(loss, wrt, allow_unused=True)
    return outs, g
