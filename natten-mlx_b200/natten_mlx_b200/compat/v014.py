"""NATTEN v0.14 operators: heads-first tensors, QK without the softmax scale, plus a
relative-position-bias table (``src/natten_mlx/compat/v014.py:192-313``).

``natten1dqkrpb(q, k, rpb, kernel_size, dilation)``: q, k ``[B, heads, L, D]``, rpb
``[heads, 2K-1]`` → logits ``[B, heads, L, K]`` with ``logits = q·k + rpb[h, pb(i) + k]`` and
``-inf`` in slots outside the sequence.  The 2-D forms take ``[B, heads, H, W, D]`` and
``[heads, 2Kh-1, 2Kw-1]``.  The reference gathers the bias on the host and adds it to the
split-QK result divided by the default scale; here the bias is added inside the QK kernel
(``natten_b200_qk_forward`` with ``bias``) at scale 1, and its gradient comes from the same
kernel family, so the functions are differentiable in q, k and rpb.

The modules are the current ones under the old argument names (``dim``; no stride, no causal
axis, no grouped heads).
"""

from __future__ import annotations

import torch

from .. import nn as _nn
from ..extras.allin1 import na1d_av_fused, na1d_qk_rpb, na2d_av_fused, na2d_qk_rpb
from ..utils.params import (check_dilation_kernel_vs_input, check_kernel_size_vs_input, normalize_kernel_size,
                            normalize_tuple_param)


def _square(kernel_size, dilation, rank, spatial):
    ks = normalize_kernel_size(kernel_size, rank)
    dl = tuple(int(d) for d in normalize_tuple_param(dilation, rank, "dilation"))
    check_kernel_size_vs_input(ks, spatial)
    check_dilation_kernel_vs_input(dl, ks, spatial)
    if len(set(ks)) != 1 or len(set(dl)) != 1:
        raise ValueError("the fused QK+RPB kernels take one kernel size and one dilation for all axes")
    return ks, dl


def natten1dqkrpb(query, key, rpb, kernel_size, dilation):
    if query.dim() != 4 or key.dim() != 4:
        raise ValueError("query and key must be [B, H, L, D]")
    ks, dl = _square(kernel_size, dilation, 1, (int(query.shape[2]),))
    if rpb.dim() != 2 or int(rpb.shape[1]) != 2 * ks[0] - 1:
        raise ValueError(f"rpb must be [heads, {2 * ks[0] - 1}] for kernel_size={ks[0]}, got {tuple(rpb.shape)}")
    logits = na1d_qk_rpb(query.transpose(1, 2), key.transpose(1, 2), rpb, ks[0], dl[0], scale=1.0)
    return logits.transpose(1, 2)


def natten1dav(attn, value, kernel_size, dilation):
    ks, dl = _square(kernel_size, dilation, 1, (int(value.shape[2]),))
    return na1d_av_fused(attn.transpose(1, 2), value.transpose(1, 2), ks[0], dl[0]).transpose(1, 2)


def natten2dqkrpb(query, key, rpb, kernel_size, dilation):
    if query.dim() != 5 or key.dim() != 5:
        raise ValueError("query and key must be [B, H, Hh, Hw, D]")
    ks, dl = _square(kernel_size, dilation, 2, (int(query.shape[2]), int(query.shape[3])))
    if rpb.dim() != 3 or int(rpb.shape[1]) != 2 * ks[0] - 1 or int(rpb.shape[2]) != 2 * ks[1] - 1:
        raise ValueError(f"rpb must be [heads, 2*Kh-1, 2*Kw-1] for the provided kernel_size; got {tuple(rpb.shape)}")
    logits = na2d_qk_rpb(query.permute(0, 2, 3, 1, 4), key.permute(0, 2, 3, 1, 4), rpb, ks[0], dl[0], scale=1.0)
    return logits.permute(0, 3, 1, 2, 4)


def natten2dav(attn, value, kernel_size, dilation):
    ks, dl = _square(kernel_size, dilation, 2, (int(value.shape[2]), int(value.shape[3])))
    out = na2d_av_fused(attn.permute(0, 2, 3, 1, 4), value.permute(0, 2, 3, 1, 4), ks[0], dl[0])
    return out.permute(0, 3, 1, 2, 4)


class NeighborhoodAttention1D(_nn.NeighborhoodAttention1D):
    def __init__(self, dim, kernel_size, dilation=1, num_heads=1, qkv_bias=True, qk_scale=None, attn_drop=0.0,
                 proj_drop=0.0, **kw):
        if dim % num_heads != 0:
            raise ValueError("dim must be divisible by num_heads")
        super().__init__(dim, num_heads, kernel_size, dilation=dilation, qkv_bias=qkv_bias, qk_scale=qk_scale or None,
                         attn_drop=attn_drop, proj_drop=proj_drop, **kw)
        self.dim = dim


class NeighborhoodAttention2D(_nn.NeighborhoodAttention2D):
    def __init__(self, dim, kernel_size, dilation=1, num_heads=1, qkv_bias=True, qk_scale=None, attn_drop=0.0,
                 proj_drop=0.0, **kw):
        if dim % num_heads != 0:
            raise ValueError("dim must be divisible by num_heads")
        super().__init__(dim, num_heads, kernel_size, dilation=dilation, qkv_bias=qkv_bias, qk_scale=qk_scale or None,
                         attn_drop=attn_drop, proj_drop=proj_drop, **kw)
        self.dim = dim


def add_natten_handle(flop_counter):
    """fvcore flop-counter hook of the old package: nothing to register here."""
    return flop_counter


__all__ = ["NeighborhoodAttention1D", "NeighborhoodAttention2D", "natten1dqkrpb", "natten1dav", "natten2dqkrpb",
           "natten2dav", "add_natten_handle"]
