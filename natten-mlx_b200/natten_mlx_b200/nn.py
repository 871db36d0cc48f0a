"""torch modules around the fused operators: the immediate callers of the hot path.

Behaviour follows the reference's MLX modules
(``src/natten_mlx/nn/na1d.py:14-154``, ``nn/na2d.py:14-154``, ``nn/na3d.py:14-158``):
channels-last input ``[B, spatial..., C]``; one fused ``qkv`` projection, or
``q_proj`` + ``kv_proj`` when ``num_kv_heads`` differs from ``num_heads``
(grouped-query attention); the fused operator on heads-last tensors
``[B, spatial..., heads, head_dim]``; with ``attn_drop > 0`` the split path
(QK → softmax → dropout → AV); with per-sample ``spatial_sizes`` the
variable-length operator; then the output projection and its dropout.

One class serves the three ranks.  The head split is a ``view`` of the projection
output: channel order ``(3, heads, head_dim)`` of the fused projection makes
q, k and v strided views of one buffer, and the operators take them without a
copy when they are already dense (q/k/v of the fused projection are not, so one
gather per tensor remains, as in the reference's ``mx.split``).
"""

from __future__ import annotations

from typing import Optional, Sequence, Union

import torch
from torch import nn

from . import functional as F
from .utils.params import normalize_kernel_size, normalize_tuple_param

_IntOrSeq = Union[int, Sequence[int]]
_BoolOrSeq = Union[bool, Sequence[bool]]

_FUSED = {1: F.na1d, 2: F.na2d, 3: F.na3d}
_QK = {1: F.na1d_qk, 2: F.na2d_qk, 3: F.na3d_qk}
_AV = {1: F.na1d_av, 2: F.na2d_av, 3: F.na3d_av}
_VARLEN = {1: F.na1d_varlen, 2: F.na2d_varlen, 3: F.na3d_varlen}
_LAYOUT = {1: "[B, L, C]", 2: "[B, H, W, C]", 3: "[B, D, H, W, C]"}


class _NeighborhoodAttention(nn.Module):
    rank = 0

    def __init__(self, embed_dim: int, num_heads: int, kernel_size: _IntOrSeq, stride: _IntOrSeq = 1,
                 dilation: _IntOrSeq = 1, is_causal: _BoolOrSeq = False, num_kv_heads: Optional[int] = None,
                 qkv_bias: bool = True, qk_scale: Optional[float] = None, attn_drop: float = 0.0,
                 proj_drop: float = 0.0, device=None, dtype=None):
        super().__init__()
        if embed_dim <= 0:
            raise ValueError(f"embed_dim must be positive, got {embed_dim}")
        if num_heads <= 0:
            raise ValueError(f"num_heads must be positive, got {num_heads}")
        if embed_dim % num_heads != 0:
            raise ValueError("embed_dim must be divisible by num_heads")
        kv_heads = num_heads if num_kv_heads is None else int(num_kv_heads)
        if kv_heads <= 0 or num_heads % kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({kv_heads})")
        rank = self.rank
        self.embed_dim, self.num_heads, self.num_kv_heads = int(embed_dim), int(num_heads), kv_heads
        self.head_dim = embed_dim // num_heads
        self.kernel_size = normalize_kernel_size(kernel_size, rank)
        self.stride = tuple(int(s) for s in normalize_tuple_param(stride, rank, "stride"))
        self.dilation = tuple(int(d) for d in normalize_tuple_param(dilation, rank, "dilation"))
        self.is_causal = tuple(bool(c) for c in normalize_tuple_param(is_causal, rank, "is_causal"))
        self.scale = float(qk_scale) if qk_scale is not None else self.head_dim ** -0.5
        kw = dict(device=device, dtype=dtype)
        if kv_heads != num_heads:
            self.q_proj = nn.Linear(embed_dim, num_heads * self.head_dim, bias=qkv_bias, **kw)
            self.kv_proj = nn.Linear(embed_dim, 2 * kv_heads * self.head_dim, bias=qkv_bias, **kw)
            self.qkv = None
        else:
            self.qkv = nn.Linear(embed_dim, 3 * embed_dim, bias=qkv_bias, **kw)
            self.q_proj = self.kv_proj = None
        self.attn_drop_rate = float(attn_drop)
        self.attn_drop = nn.Dropout(self.attn_drop_rate) if self.attn_drop_rate > 0.0 else None
        self.proj = nn.Linear(embed_dim, embed_dim, **kw)
        self.proj_drop_rate = float(proj_drop)
        self.proj_drop = nn.Dropout(self.proj_drop_rate) if self.proj_drop_rate > 0.0 else None

    def _heads(self, x: torch.Tensor):
        lead = tuple(x.shape[:-1])
        if self.qkv is not None:
            qkv = self.qkv(x).view(*lead, 3, self.num_heads, self.head_dim)
            return qkv.select(-3, 0), qkv.select(-3, 1), qkv.select(-3, 2)
        q = self.q_proj(x).view(*lead, self.num_heads, self.head_dim)
        kv = self.kv_proj(x).view(*lead, 2, self.num_kv_heads, self.head_dim)
        return q, kv.select(-3, 0), kv.select(-3, 1)

    def forward(self, x: torch.Tensor, spatial_sizes: Optional[torch.Tensor] = None) -> torch.Tensor:
        rank = self.rank
        if x.dim() != rank + 2:
            raise ValueError(f"Expected input shape {_LAYOUT[rank]}, got {tuple(x.shape)}")
        if x.shape[-1] != self.embed_dim:
            raise ValueError(f"Input channel dim ({x.shape[-1]}) must match embed_dim ({self.embed_dim})")
        q, k, v = self._heads(x)
        if spatial_sizes is not None:
            out = _VARLEN[rank](q, k, v, spatial_sizes, kernel_size=self.kernel_size, dilation=self.dilation,
                                scale=self.scale)
        elif self.attn_drop is not None:
            logits = _QK[rank](q, k, kernel_size=self.kernel_size, dilation=self.dilation, stride=self.stride,
                               is_causal=self.is_causal, scale=self.scale)
            attn = self.attn_drop(torch.softmax(logits, dim=-1))
            out = _AV[rank](attn, v, kernel_size=self.kernel_size, dilation=self.dilation, stride=self.stride,
                            is_causal=self.is_causal)
        else:
            out = _FUSED[rank](q, k, v, kernel_size=self.kernel_size, stride=self.stride, dilation=self.dilation,
                               is_causal=self.is_causal, scale=self.scale)
        out = self.proj(out.reshape(*out.shape[:-2], self.embed_dim))
        return out if self.proj_drop is None else self.proj_drop(out)

    def extra_repr(self) -> str:
        return (f"embed_dim={self.embed_dim}, num_heads={self.num_heads}, num_kv_heads={self.num_kv_heads}, "
                f"kernel_size={self.kernel_size}, stride={self.stride}, dilation={self.dilation}, "
                f"is_causal={self.is_causal}")


class NeighborhoodAttention1D(_NeighborhoodAttention):
    """Input ``[B, L, C]`` → output ``[B, ceil(L / stride), C]``; ``forward(x, seq_lens)`` for ragged batches."""
    rank = 1


class NeighborhoodAttention2D(_NeighborhoodAttention):
    """Input ``[B, H, W, C]`` → output ``[B, ceil(H / stride_h), ceil(W / stride_w), C]``."""
    rank = 2


class NeighborhoodAttention3D(_NeighborhoodAttention):
    """Input ``[B, D, H, W, C]`` → output with every spatial extent divided (rounding up) by its stride."""
    rank = 3


__all__ = ["NeighborhoodAttention1D", "NeighborhoodAttention2D", "NeighborhoodAttention3D"]
