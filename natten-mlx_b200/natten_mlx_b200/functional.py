"""Public functional API: same names, arguments, defaults and ``ValueError``
conditions as src/natten_mlx/functional.py:207-844, over torch CUDA tensors.

Differences in how the work is done, not in what is computed:

* GQA/MQA never materialises repeated K/V heads; the kernels index the KV head
  as ``h // (H_q / H_kv)`` (the reference repeats, functional.py:29-33).
* ``return_lse`` and ``additional_keys/values`` run inside the one fused
  kernel of either family (window slots and extra tokens share a softmax: on
  the tensor-core kernels the extra tokens are one more chunk of keys after
  the key box) instead of the split-QK -> softmax -> AV -> dense attention ->
  merge chain of functional.py:276-292; the results are the same function of
  the inputs.
* A kernel that covers the whole extent takes the same fused kernel (the
  reference routes it to a dense-attention library call, functional.py:141-187).
* The varlen ops also accept GQA, ``return_lse`` and extra tokens, and take
  ``host_sizes`` (a host copy of the sizes): with it a bf16/fp16 batch runs
  on the tensor-core kernels in one launch per kernel without a
  device-to-host copy.
"""

from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from . import autograd as _ag
from .utils.params import (check_dilation_kernel_vs_input, check_kernel_size_vs_input,
                           check_stride_vs_kernel, normalize_kernel_size, normalize_tuple_param)

_LAYOUTS = {1: "[B, L, H, D]", 2: "[B, H, W, heads, dim]", 3: "[B, D, H, W, heads, dim]"}


def _validate_qkv(query, key, value, rank: int) -> int:
    """Shape checks of functional.py:36-68; returns H_q / H_kv."""
    nd = rank + 3
    if query.dim() != nd or key.dim() != nd or value.dim() != nd:
        raise ValueError(f"na{rank}d expects query/key/value with shape {_LAYOUTS[rank]}.")
    sq, sk, sv = tuple(query.shape[1:-2]), tuple(key.shape[1:-2]), tuple(value.shape[1:-2])
    if sq != sk or sq != sv:
        raise ValueError(f"Spatial dimensions must match: Q={sq}, K={sk}, V={sv}.")
    if query.shape[0] != key.shape[0] or query.shape[0] != value.shape[0]:
        raise ValueError("Batch dimensions must match.")
    if query.shape[-1] != key.shape[-1]:
        raise ValueError(f"Head dim must match: Q has {query.shape[-1]}, K has {key.shape[-1]}.")
    if key.shape[-2] != value.shape[-2]:
        raise ValueError("K and V must have same number of heads.")
    if key.shape[-1] != value.shape[-1]:
        raise ValueError(f"Head dim must match: K has {key.shape[-1]}, V has {value.shape[-1]}.")
    if query.shape[-2] % key.shape[-2] != 0:
        raise ValueError(
            f"heads_q ({query.shape[-2]}) must be divisible by heads_kv ({key.shape[-2]}) for GQA.")
    return query.shape[-2] // key.shape[-2]


def _validate_additional_kv(query, key, additional_keys, additional_values):
    """Checks of functional.py:107-138 (the tokens keep their H_kv heads here)."""
    if additional_keys is None and additional_values is None:
        return None, None
    if additional_keys is None or additional_values is None:
        raise ValueError("additional_keys and additional_values must both be provided or both None.")
    if additional_keys.dim() != 4 or additional_values.dim() != 4:
        raise ValueError("additional_keys/additional_values must be 4D: [B, N_extra, heads_kv, dim].")
    if additional_keys.shape[0] != query.shape[0]:
        raise ValueError("additional_keys batch must match query batch.")
    if additional_values.shape[0] != query.shape[0]:
        raise ValueError("additional_values batch must match query batch.")
    if additional_keys.shape[-1] != query.shape[-1]:
        raise ValueError("additional_keys head dim must match query head dim.")
    if additional_values.shape[-1] != query.shape[-1]:
        raise ValueError("additional_values head dim must match query head dim.")
    if additional_keys.shape[-2] != additional_values.shape[-2]:
        raise ValueError("additional_keys and additional_values must have same number of heads.")
    if additional_keys.shape[1] != additional_values.shape[1]:
        raise ValueError("additional_keys and additional_values must have same N_extra.")
    if additional_keys.shape[-2] != key.shape[-2]:
        raise ValueError("additional_keys heads must match the key/value heads.")
    return additional_keys, additional_values


def _normalize(rank, spatial, kernel_size, stride, dilation, is_causal):
    ks = normalize_kernel_size(kernel_size, rank)
    st = normalize_tuple_param(stride, rank, "stride")
    dl = normalize_tuple_param(dilation, rank, "dilation")
    ca = tuple(bool(c) for c in normalize_tuple_param(is_causal, rank, "is_causal"))
    check_kernel_size_vs_input(ks, spatial)
    check_stride_vs_kernel(st, ks)
    check_dilation_kernel_vs_input(dl, ks, spatial)
    return ks, st, dl, ca


def _na(rank, query, key, value, kernel_size, stride, dilation, is_causal, scale, return_lse,
        additional_keys, additional_values):
    _validate_qkv(query, key, value, rank)
    add_k, add_v = _validate_additional_kv(query, key, additional_keys, additional_values)
    spatial = tuple(query.shape[1:-2])
    ks, st, dl, ca = _normalize(rank, spatial, kernel_size, stride, dilation, is_causal)
    if add_k is not None and any(s != 1 for s in st) and not all(
            -(-e // s) == e for e, s in zip(spatial, st)):
        # the reference's dense branch runs on every query and its merge then
        # rejects the shape mismatch (functional.py:289-292, merge.py:41-45)
        raise ValueError("additional_keys/values with a strided output: shape does not match output 0")
    scale_value = query.shape[-1] ** -0.5 if scale is None else float(scale)
    if all(k >= e for k, e in zip(ks, spatial)) and all(s == 1 for s in st) and not any(ca):
        # kernel covers every axis: dense attention over the extent (functional.py:141-143, 271)
        ca = (2,) * rank
    out, lse = _ag.fused_with_grad(query, key, value, ks, st, dl, ca, scale_value, add_k, add_v)
    return (out, lse) if return_lse else out


def na1d(query, key, value, kernel_size: Union[int, Tuple[int]], stride=1, dilation=1, is_causal=False,
         scale: Optional[float] = None, return_lse: bool = False,
         additional_keys: Optional[torch.Tensor] = None, additional_values: Optional[torch.Tensor] = None):
    """1D neighborhood attention.  query ``[B, L, H_q, D]``, key/value ``[B, L, H_kv, D]``.

    Returns ``[B, ceil(L/stride), H_q, D]``, or ``(output, lse)`` with
    ``lse [B, ceil(L/stride), H_q]`` float32 when ``return_lse`` is set.
    """
    return _na(1, query, key, value, kernel_size, stride, dilation, is_causal, scale, return_lse,
               additional_keys, additional_values)


def na2d(query, key, value, kernel_size, stride=1, dilation=1, is_causal=False,
         scale: Optional[float] = None, return_lse: bool = False,
         additional_keys: Optional[torch.Tensor] = None, additional_values: Optional[torch.Tensor] = None):
    """2D neighborhood attention over ``[B, H, W, heads, D]`` tensors."""
    return _na(2, query, key, value, kernel_size, stride, dilation, is_causal, scale, return_lse,
               additional_keys, additional_values)


def na3d(query, key, value, kernel_size, stride=1, dilation=1, is_causal=False,
         scale: Optional[float] = None, return_lse: bool = False,
         additional_keys: Optional[torch.Tensor] = None, additional_values: Optional[torch.Tensor] = None):
    """3D neighborhood attention over ``[B, D, H, W, heads, dim]`` tensors."""
    return _na(3, query, key, value, kernel_size, stride, dilation, is_causal, scale, return_lse,
               additional_keys, additional_values)


# ---------------------------------------------------------------------------
# split ops (functional.py:476-634)
# ---------------------------------------------------------------------------

def _qk(rank, query, key, kernel_size, dilation, stride, is_causal, scale):
    _validate_qkv(query, key, key, rank)
    spatial = tuple(query.shape[1:-2])
    ks, st, dl, ca = _normalize(rank, spatial, kernel_size, stride, dilation, is_causal)
    return getattr(_ag, f"na{rank}d_qk_with_grad")(query, key, ks, st, dl, ca, scale)


def _av(rank, attn, value, kernel_size, dilation, stride, is_causal):
    nd = rank + 3
    if attn.dim() != nd or value.dim() != nd:
        raise ValueError(f"attn and value must be {nd}D for na{rank}d_av")
    if attn.shape[0] != value.shape[0] or attn.shape[-2] % value.shape[-2] != 0:
        raise ValueError("attn and value must match batch and heads dimensions; "
                         f"got {tuple(attn.shape)} and {tuple(value.shape)}")
    spatial = tuple(value.shape[1:-2])
    ks, st, dl, ca = _normalize(rank, spatial, kernel_size, stride, dilation, is_causal)
    return getattr(_ag, f"na{rank}d_av_with_grad")(attn, value, ks, st, dl, ca)


def na1d_qk(query, key, kernel_size, dilation=1, *, stride=1, is_causal=False, scale=None):
    """Separate 1D query-key logits, ``[B, ceil(L/stride), H, K]``; invalid slots are ``-inf``."""
    return _qk(1, query, key, kernel_size, dilation, stride, is_causal, scale)


def na2d_qk(query, key, kernel_size, dilation=1, *, stride=1, is_causal=False, scale=None):
    """Separate 2D query-key logits, ``[B, Oh, Ow, heads, Kh*Kw]``."""
    return _qk(2, query, key, kernel_size, dilation, stride, is_causal, scale)


def na3d_qk(query, key, kernel_size, dilation=1, *, stride=1, is_causal=False, scale=None):
    """Separate 3D query-key logits, ``[B, Od, Oh, Ow, heads, Kd*Kh*Kw]``."""
    return _qk(3, query, key, kernel_size, dilation, stride, is_causal, scale)


def na1d_av(attn, value, kernel_size, dilation=1, *, stride=1, is_causal=False):
    """Separate 1D attention-value product; attn ``[B, ceil(L/stride), H, K]``."""
    return _av(1, attn, value, kernel_size, dilation, stride, is_causal)


def na2d_av(attn, value, kernel_size, dilation=1, *, stride=1, is_causal=False):
    """Separate 2D attention-value product."""
    return _av(2, attn, value, kernel_size, dilation, stride, is_causal)


def na3d_av(attn, value, kernel_size, dilation=1, *, stride=1, is_causal=False):
    """Separate 3D attention-value product."""
    return _av(3, attn, value, kernel_size, dilation, stride, is_causal)


# ---------------------------------------------------------------------------
# variable-size batches (functional.py:637-828)
# ---------------------------------------------------------------------------

def _validate_sizes(sizes, batch, max_spatial, ks, rank, host_sizes=None):
    """Checks of functional.py:637-694.  ``sizes`` may live on the GPU; the
    range checks read ``host_sizes`` when given, else copy ``sizes`` to the host.
    Returns the sizes tensor and the host list of per-sample extents."""
    if not torch.is_tensor(sizes):
        sizes = torch.as_tensor(sizes)
    if rank == 1:
        if sizes.dim() != 1 or sizes.shape[0] != batch:
            raise ValueError(f"seq_lens must be a 1-D array of length B={batch}, got shape {tuple(sizes.shape)}.")
        name = "seq_lens"
    else:
        if sizes.dim() != 2 or sizes.shape[0] != batch or sizes.shape[1] != rank:
            raise ValueError(f"spatial_sizes must be a [B, {rank}] array, got shape {tuple(sizes.shape)}.")
        name = "spatial_sizes"
    if sizes.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"{name} must be int32 or int64, got {sizes.dtype}.")
    host = torch.as_tensor(host_sizes) if host_sizes is not None else sizes.detach().cpu()
    host = host.reshape(batch, rank)
    for a in range(rank):
        lo, hi = int(host[:, a].min()), int(host[:, a].max())
        if rank == 1:
            if lo < ks[a]:
                raise ValueError(f"All seq_lens must be >= kernel_size ({ks[a]}), but min(seq_lens)={lo}.")
            if hi > max_spatial[a]:
                raise ValueError(f"All seq_lens must be <= L_max ({max_spatial[a]}), but max(seq_lens)={hi}.")
        else:
            if lo < ks[a]:
                raise ValueError(f"All spatial_sizes[:,{a}] must be >= kernel_size[{a}] ({ks[a]}), but min={lo}.")
            if hi > max_spatial[a]:
                raise ValueError(
                    f"All spatial_sizes[:,{a}] must be <= max_spatial[{a}] ({max_spatial[a]}), but max={hi}.")
    return sizes, [tuple(int(x) for x in row) for row in host.tolist()]


def _varlen(rank, query, key, value, sizes, kernel_size, dilation, scale, return_lse, additional_keys,
            additional_values, host_sizes):
    nd = rank + 3
    if query.dim() != nd or key.dim() != nd or value.dim() != nd:
        raise ValueError(f"na{rank}d_varlen expects query/key/value with shape {_LAYOUTS[rank]}.")
    if key.shape != value.shape or query.shape[:-2] != key.shape[:-2] or query.shape[-1] != key.shape[-1] \
            or query.shape[-2] % key.shape[-2] != 0:
        raise ValueError("query, key, and value must have identical shapes "
                         "(key/value may carry fewer heads that divide the query heads).")
    add_k, add_v = _validate_additional_kv(query, key, additional_keys, additional_values)
    ks = normalize_kernel_size(kernel_size, rank)
    dl = normalize_tuple_param(dilation, rank, "dilation")
    for a, d in enumerate(dl):
        if not isinstance(d, int) or d <= 0:
            raise ValueError(f"dilation[{a}] must be a positive int, got {d!r}")
    sizes, host = _validate_sizes(sizes, query.shape[0], tuple(query.shape[1:-2]), ks, rank, host_sizes)
    scale_value = query.shape[-1] ** -0.5 if scale is None else float(scale)
    one, no = (1,) * rank, (False,) * rank
    out, lse = _ag.fused_with_grad(query, key, value, ks, one, dl, no, scale_value, add_k, add_v,
                                   sizes.to(device=query.device, dtype=torch.int32), host)
    return (out, lse) if return_lse else out


def na1d_varlen(query, key, value, seq_lens, kernel_size, dilation=1, scale: Optional[float] = None, *,
                return_lse: bool = False, additional_keys=None, additional_values=None, host_sizes=None):
    """Variable-length 1D attention: sample ``b`` attends within its first
    ``seq_lens[b]`` positions of the padded ``[B, L_max, H, D]`` tensors and the
    padding comes back as zeros."""
    return _varlen(1, query, key, value, seq_lens, kernel_size, dilation, scale, return_lse,
                   additional_keys, additional_values, host_sizes)


def na2d_varlen(query, key, value, spatial_sizes, kernel_size, dilation=1, scale: Optional[float] = None, *,
                return_lse: bool = False, additional_keys=None, additional_values=None, host_sizes=None):
    """Variable-size 2D attention; ``spatial_sizes`` is ``[B, 2]`` (H_b, W_b)."""
    return _varlen(2, query, key, value, spatial_sizes, kernel_size, dilation, scale, return_lse,
                   additional_keys, additional_values, host_sizes)


def na3d_varlen(query, key, value, spatial_sizes, kernel_size, dilation=1, scale: Optional[float] = None, *,
                return_lse: bool = False, additional_keys=None, additional_values=None, host_sizes=None):
    """Variable-size 3D attention; ``spatial_sizes`` is ``[B, 3]`` (D_b, H_b, W_b)."""
    return _varlen(3, query, key, value, spatial_sizes, kernel_size, dilation, scale, return_lse,
                   additional_keys, additional_values, host_sizes)


__all__ = [
    "na1d", "na1d_varlen", "na2d", "na2d_varlen", "na3d", "na3d_varlen",
    "na1d_qk", "na1d_av", "na2d_qk", "na2d_av", "na3d_qk", "na3d_av",
]
