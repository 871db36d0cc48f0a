"""DiNAT-style ops: QK with relative position bias, and AV
(src/natten_mlx/extras/allin1/__init__.py:40-180).

Heads-last layout, scalar ``kernel_size`` and ``dilation``, stride 1, no
causal axis.  ``scale`` multiplies the QK product only; the bias is added
unscaled, as in the reference (``query = query * scale`` before the product,
__init__.py:61-62).  Unlike the reference these ops are differentiable
(q, k, rpb, attn, v all receive gradients).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import autograd as _ag


def _qk_rpb(rank, query, key, rpb, kernel_size, dilation, scale):
    k = int(kernel_size)
    d = int(dilation)
    if rpb is not None:
        want = (query.shape[-2],) + (2 * k - 1,) * rank
        if tuple(rpb.shape) != want:
            raise ValueError(f"rpb must have shape {want}, got {tuple(rpb.shape)}")
        rpb = rpb.to(device=query.device, dtype=torch.float32)
    for a in range(rank):
        if k * d > query.shape[1 + a]:
            raise ValueError(
                f"kernel_size * dilation must be <= axis length; got kernel_size={k}, dilation={d}, "
                f"axis length={query.shape[1 + a]}")
    return _ag.qk_bias_with_grad(query, key, rpb, (k,) * rank, (d,) * rank, 1.0 if scale is None else float(scale))


def na1d_qk_rpb(query, key, rpb: Optional[torch.Tensor], kernel_size: int, dilation: int = 1, *,
                scale: Optional[float] = None):
    """Fused 1D QK + RPB.  query/key ``[B, L, H, D]``, rpb ``[H, 2K-1]`` or None -> ``[B, L, H, K]``."""
    if query.dim() != 4:
        raise ValueError(f"query must be 4D [B, L, H, D], got shape {tuple(query.shape)}")
    return _qk_rpb(1, query, key, rpb, kernel_size, dilation, scale)


def na2d_qk_rpb(query, key, rpb: Optional[torch.Tensor], kernel_size: int, dilation: int = 1, *,
                scale: Optional[float] = None):
    """Fused 2D QK + RPB.  query/key ``[B, Hh, Hw, H, D]``, rpb ``[H, 2K-1, 2K-1]`` or None -> ``[B, Hh, Hw, H, K*K]``."""
    if query.dim() != 5:
        raise ValueError(f"query must be 5D [B, Hh, Hw, H, D], got shape {tuple(query.shape)}")
    return _qk_rpb(2, query, key, rpb, kernel_size, dilation, scale)


def na1d_av_fused(attn, value, kernel_size: int, dilation: int = 1):
    """Fused 1D AV.  attn ``[B, L, H, K]``, value ``[B, L, H, D]`` -> ``[B, L, H, D]``."""
    if attn.dim() != 4 or value.dim() != 4:
        raise ValueError("attn and value must be 4D for na1d_av_fused")
    return _ag.na1d_av_with_grad(attn, value, (int(kernel_size),), (1,), (int(dilation),), (False,))


def na2d_av_fused(attn, value, kernel_size: int, dilation: int = 1):
    """Fused 2D AV.  attn ``[B, Hh, Hw, H, K*K]``, value ``[B, Hh, Hw, H, D]`` -> ``[B, Hh, Hw, H, D]``."""
    if attn.dim() != 5 or value.dim() != 5:
        raise ValueError("attn and value must be 5D for na2d_av_fused")
    k, d = int(kernel_size), int(dilation)
    return _ag.na2d_av_with_grad(attn, value, (k, k), (1, 1), (d, d), (False, False))


def _qkv_fused(rank, query, key, value, rpb, kernel_size, dilation, scale):
    from .._core import cuda as _backend
    k, d = int(kernel_size), int(dilation)
    if query.dim() != rank + 3 or key.shape != query.shape[:-2] + key.shape[-2:] or value.shape != key.shape:
        raise ValueError(f"query/key/value must be {rank + 3}D heads-last tensors of matching shape")
    if rpb is not None:
        want = (query.shape[-2],) + (2 * k - 1,) * rank
        if tuple(rpb.shape) != want:
            raise ValueError(f"rpb must have shape {want}, got {tuple(rpb.shape)}")
    for a in range(rank):
        if k * d > query.shape[1 + a]:
            raise ValueError(
                f"kernel_size * dilation must be <= axis length; got kernel_size={k}, dilation={d}, "
                f"axis length={query.shape[1 + a]}")
    with torch.no_grad():
        return _backend.qk_bias_av_forward(query, key, value, (k,) * rank, (d,) * rank,
                                           1.0 if scale is None else float(scale), bias=rpb)


def na1d_qkv_fused(query, key, value, rpb: Optional[torch.Tensor], kernel_size: int, dilation: int = 1, *,
                   scale: Optional[float] = None):
    """QK + RPB -> softmax -> AV of 1D neighborhood attention in one launch (inference: no gradients).
    Equals ``na1d_av_fused(softmax(na1d_qk_rpb(q, k, rpb)), v)`` without the logits ever reaching memory
    (natten2d_qkv_fused of the reference, src/natten_mlx/extras/allin1/functional_metal.py:2130-2170)."""
    return _qkv_fused(1, query, key, value, rpb, kernel_size, dilation, scale)


def na2d_qkv_fused(query, key, value, rpb: Optional[torch.Tensor], kernel_size: int, dilation: int = 1, *,
                   scale: Optional[float] = None):
    """QK + RPB -> softmax -> AV of 2D neighborhood attention in one launch (inference: no gradients)."""
    return _qkv_fused(2, query, key, value, rpb, kernel_size, dilation, scale)


__all__ = ["na1d_qk_rpb", "na1d_av_fused", "na2d_qk_rpb", "na2d_av_fused", "na1d_qkv_fused", "na2d_qkv_fused"]
