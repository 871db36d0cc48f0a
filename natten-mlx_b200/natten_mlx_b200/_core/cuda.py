"""The ``cuda`` backend: the backend-module protocol of the reference's
dispatcher (src/natten_mlx/_core/ops.py:49-135) implemented on the C ABI.

Every function takes contiguous-able CUDA tensors in heads-last layout and
launches on torch's current stream.  There is no CPU path: a CPU tensor or a
missing library raises.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import ctypes

import torch

from .. import _lib

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}

# Kernel family used by the fused entry points ("auto", "simt", "tcgen05").
_PATHS = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tcgen05": _lib.PATH_TCGEN05}
_fused_path = "auto"


def set_fused_path(name: str) -> None:
    """Select the kernel family of the fused ops: "auto", "simt" or "tcgen05"."""
    global _fused_path
    if name not in _PATHS:
        raise ValueError(f"Unknown fused path {name!r}. Expected one of {sorted(_PATHS)}")
    _fused_path = name


def get_fused_path() -> str:
    return _fused_path


def is_available() -> bool:
    try:
        _lib.load()
    except (ImportError, OSError, AttributeError):
        return False
    return torch.cuda.is_available()


@dataclass(frozen=True)
class Slab:
    """A slab of a larger volume: where the local query / key tensors sit in
    global coordinates (used by leading-axis sharding with K/V halo planes)."""
    global_extent: Tuple[int, ...]
    q_offset: Tuple[int, ...]
    kv_offset: Tuple[int, ...]


def _prep(*tensors: torch.Tensor):
    t0 = tensors[0]
    if not t0.is_cuda:
        raise RuntimeError("natten_mlx_b200 runs on CUDA tensors only (there is no CPU path)")
    if t0.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {t0.dtype}; expected float32, float16 or bfloat16")
    out = []
    for t in tensors:
        if t is None:
            out.append(None)
            continue
        if t.device != t0.device or t.dtype != t0.dtype:
            raise ValueError("all tensors must share device and dtype")
        t = t.contiguous()
        if t.data_ptr() % 16 != 0:      # a dense view at an odd storage offset: the kernels need 16-byte aligned bases
            t = t.clone()
        out.append(t)
    return out


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def _scale(scale, head_dim):
    return head_dim ** -0.5 if scale is None else float(scale)


def _out_shape(extent, stride):
    return tuple(-(-e // s) for e, s in zip(extent, stride))


def _sizes_tensor(sizes, batch, rank, device):
    if sizes is None:
        return None
    s = sizes if torch.is_tensor(sizes) else torch.as_tensor(sizes)
    return s.to(device=device, dtype=torch.int32).reshape(batch, rank).contiguous()


def _geom(q_like, kv_like, rank, ks, st, dl, ca, scale, *, heads_q=None, n_extra=0, sizes=None,
          slab: Optional[Slab] = None, path=None, host_sizes=None):
    extent = tuple(q_like.shape[1:1 + rank])
    kv_extent = tuple(kv_like.shape[1:1 + rank])
    kw = {}
    if slab is not None:
        kw = dict(q_extent=extent, kv_extent=kv_extent, q_offset=slab.q_offset, kv_offset=slab.kv_offset)
        extent = tuple(slab.global_extent)
    elif kv_extent != extent:
        raise ValueError(f"Spatial dimensions must match: Q={extent}, K={kv_extent}.")
    return _lib.make_geom(
        rank, q_like.shape[0], heads_q if heads_q is not None else q_like.shape[-2], kv_like.shape[-2],
        kv_like.shape[-1], _DTYPES[kv_like.dtype], extent, ks, st, dl, ca, scale, n_extra=n_extra,
        path=_PATHS[_fused_path] if path is None else _PATHS[path],
        extents_ptr=0 if sizes is None else sizes.data_ptr(),
        host_extents=None if sizes is None else host_sizes, **kw)


# ---------------------------------------------------------------------------
# split operators
# ---------------------------------------------------------------------------

def qk_forward(q, k, ks, st, dl, ca, scale, bias=None, slab=None):
    rank = q.dim() - 3
    q, k = _prep(q, k)
    g = _geom(q, k, rank, ks, st, dl, ca, _scale(scale, q.shape[-1]), slab=slab)
    outs = _out_shape(q.shape[1:1 + rank], st)
    kvol = 1
    for x in ks:
        kvol *= x
    logits = torch.empty((q.shape[0],) + outs + (q.shape[-2], kvol), dtype=q.dtype, device=q.device)
    if bias is not None:
        bias = bias.to(device=q.device, dtype=torch.float32).contiguous()
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().natten_b200_qk_forward(g, _ptr(q), _ptr(k), _ptr(bias), _ptr(logits), _stream(q)))
    return logits


def qk_backward(q, k, grad_attn, ks, st, dl, ca, scale, want_dbias_shape=None, slab=None):
    rank = q.dim() - 3
    q, k, grad_attn = _prep(q, k, grad_attn)
    g = _geom(q, k, rank, ks, st, dl, ca, _scale(scale, q.shape[-1]), slab=slab)
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    dbias = None
    if want_dbias_shape is not None:
        dbias = torch.zeros(want_dbias_shape, dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().natten_b200_qk_backward(g, _ptr(q), _ptr(k), _ptr(grad_attn), _ptr(dq), _ptr(dk),
                                                       _ptr(dbias), _stream(q)))
    return (dq, dk) if dbias is None else (dq, dk, dbias)


def qk_bias_av_forward(q, k, v, ks, dl, scale, bias=None, return_lse=False):
    """QK + bias -> softmax -> AV in one launch (forward only, stride 1, no causal axis)."""
    rank = q.dim() - 3
    q, k, v = _prep(q, k, v)
    one, no = (1,) * rank, (False,) * rank
    g = _geom(q, k, rank, ks, one, dl, no, _scale(scale, q.shape[-1]))
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:-1], dtype=torch.float32, device=q.device) if return_lse else None
    if bias is not None:
        bias = bias.to(device=q.device, dtype=torch.float32).contiguous()
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().natten_b200_qk_bias_av_forward(g, _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(out),
                                                              _ptr(lse), _stream(q)))
    return (out, lse) if return_lse else out


def _check_attn(attn, v, rank, ks, st):
    kvol = 1
    for x in ks:
        kvol *= x
    if attn.shape[-1] != kvol:
        raise ValueError(
            f"attn neighborhood dimension must equal the kernel volume; got {attn.shape[-1]} vs {kvol}")
    outs = _out_shape(v.shape[1:1 + rank], st)
    if tuple(attn.shape[1:1 + rank]) != outs:
        raise ValueError(
            f"attn spatial dimensions must match ceil(input/stride); got {tuple(attn.shape[1:1 + rank])} vs {outs}")
    if attn.shape[-2] % v.shape[-2] != 0:
        raise ValueError("attn heads must be divisible by value heads")


def av_forward(attn, v, ks, st, dl, ca):
    rank = v.dim() - 3
    attn, v = _prep(attn, v)
    _check_attn(attn, v, rank, ks, st)
    g = _geom(v, v, rank, ks, st, dl, ca, 1.0, heads_q=attn.shape[-2])
    out = torch.empty(attn.shape[:-1] + (v.shape[-1],), dtype=v.dtype, device=v.device)
    with torch.cuda.device(v.device):
        _lib.check(_lib.load().natten_b200_av_forward(g, _ptr(attn), _ptr(v), _ptr(out), _stream(v)))
    return out


def av_backward(attn, v, grad_out, ks, st, dl, ca):
    rank = v.dim() - 3
    attn, v, grad_out = _prep(attn, v, grad_out)
    _check_attn(attn, v, rank, ks, st)
    g = _geom(v, v, rank, ks, st, dl, ca, 1.0, heads_q=attn.shape[-2])
    dattn, dv = torch.empty_like(attn), torch.empty_like(v)
    with torch.cuda.device(v.device):
        _lib.check(_lib.load().natten_b200_av_backward(g, _ptr(attn), _ptr(v), _ptr(grad_out), _ptr(dattn), _ptr(dv),
                                                       _stream(v)))
    return dattn, dv


# ---------------------------------------------------------------------------
# fused operator
# ---------------------------------------------------------------------------

def _host_sizes(sizes, host_sizes, batch, rank):
    """Per-sample extents as a host list of ``rank``-tuples: the caller's copy, or one read back from the device
    tensor (a synchronising copy; pass ``host_sizes`` to avoid it)."""
    if sizes is None:
        return None
    if host_sizes is None:
        host_sizes = (sizes.detach().cpu() if torch.is_tensor(sizes) else torch.as_tensor(sizes)).reshape(batch, rank).tolist()
    return [tuple(int(x) for x in (s if isinstance(s, (list, tuple)) else (s,))) for s in host_sizes]


def fused_forward(q, k, v, ks, st, dl, ca, scale, *, k_extra=None, v_extra=None, sizes=None,
                  slab: Optional[Slab] = None, path=None, host_sizes=None, out=None, lse=None):
    """Returns (out, lse); lse is float32 [B, out..., H_q].  With per-sample ``sizes`` the padding of both is zero.
    ``out`` / ``lse`` (both or neither): dense tensors to write into instead of new ones."""
    rank = q.dim() - 3
    q, k, v, k_extra, v_extra = _prep(q, k, v, k_extra, v_extra)
    n_extra = 0 if k_extra is None else k_extra.shape[1]
    sizes_t = _sizes_tensor(sizes, q.shape[0], rank, q.device)
    g = _geom(q, k, rank, ks, st, dl, ca, _scale(scale, q.shape[-1]), n_extra=n_extra, sizes=sizes_t,
              slab=slab, path=path, host_sizes=_host_sizes(sizes, host_sizes, q.shape[0], rank))
    outs = _out_shape(q.shape[1:1 + rank], st)
    # variable-size batches: the tensor-core kernels never touch rows outside a sample, so they start from zeros
    alloc = torch.empty if sizes is None else torch.zeros
    if out is not None:
        want = (q.shape[0],) + outs + tuple(q.shape[-2:])
        if (tuple(out.shape) != want or tuple(lse.shape) != want[:-1] or not out.is_contiguous() or not lse.is_contiguous()
                or out.dtype != q.dtype or lse.dtype != torch.float32 or sizes is not None):
            raise ValueError("fused_forward: out / lse must be dense tensors of the result's shapes and dtypes")
    else:
        out = alloc((q.shape[0],) + outs + tuple(q.shape[-2:]), dtype=q.dtype, device=q.device)
        lse = alloc((q.shape[0],) + outs + (q.shape[-2],), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().natten_b200_fused_forward(g, _ptr(q), _ptr(k), _ptr(v), _ptr(k_extra), _ptr(v_extra),
                                                         _ptr(out), _ptr(lse), _stream(q)))
    return out, lse


def fused_backward(q, k, v, out, lse, grad_out, grad_lse, ks, st, dl, ca, scale, *, k_extra=None,
                   v_extra=None, sizes=None, slab: Optional[Slab] = None, path=None, host_sizes=None, halo_out=None):
    """Returns (dq, dk, dv, dk_extra, dv_extra); the last two are None without extra tokens.

    ``halo_out`` = (planes_below, planes_above, dk_below, dv_below, dk_above, dv_above) with raw addresses sends
    the gradients of a slab's halo planes there from inside the dK/dV kernel (tensor-core kernels only; see
    ``natten_b200_fused_backward_halo``); those planes of the returned dk / dv are then left unwritten."""
    rank = q.dim() - 3
    q, k, v, k_extra, v_extra, out, grad_out = _prep(q, k, v, k_extra, v_extra, out, grad_out)
    n_extra = 0 if k_extra is None else k_extra.shape[1]
    sizes_t = _sizes_tensor(sizes, q.shape[0], rank, q.device)
    g = _geom(q, k, rank, ks, st, dl, ca, _scale(scale, q.shape[-1]), n_extra=n_extra, sizes=sizes_t,
              slab=slab, path=path, host_sizes=_host_sizes(sizes, host_sizes, q.shape[0], rank))
    lse = lse.contiguous()
    if grad_lse is not None:
        grad_lse = grad_lse.to(torch.float32).contiguous()
    alloc = torch.empty_like if sizes is None else torch.zeros_like     # see fused_forward
    dq, dk, dv = alloc(q), alloc(k), alloc(v)
    dke = None if k_extra is None else torch.empty_like(k_extra)
    dve = None if v_extra is None else torch.empty_like(v_extra)
    lib = _lib.load()
    nbytes = int(lib.natten_b200_fused_backward_scratch_bytes(g))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        if halo_out is not None:
            halo = _lib.HaloOut(int(halo_out[0]), int(halo_out[1]), *[int(x) if x else None for x in halo_out[2:6]])
            _lib.check(lib.natten_b200_fused_backward_halo(
                g, _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), _ptr(grad_out), _ptr(grad_lse), _ptr(dq), _ptr(dk),
                _ptr(dv), _ptr(scratch), nbytes, ctypes.byref(halo), _stream(q)))
            return dq, dk, dv, dke, dve
        _lib.check(lib.natten_b200_fused_backward(
            g, _ptr(q), _ptr(k), _ptr(v), _ptr(k_extra), _ptr(v_extra), _ptr(out), _ptr(lse), _ptr(grad_out),
            _ptr(grad_lse), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dke), _ptr(dve), _ptr(scratch), nbytes, _stream(q)))
    return dq, dk, dv, dke, dve


# ---------------------------------------------------------------------------
# merge
# ---------------------------------------------------------------------------

def merge_forward(o0, l0, o1, l1):
    o0, o1 = _prep(o0, o1)
    l0, l1 = l0.to(torch.float32).contiguous(), l1.to(torch.float32).contiguous()
    out = torch.empty_like(o0)
    lse = torch.empty_like(l0)
    rows = l0.numel()
    with torch.cuda.device(o0.device):
        _lib.check(_lib.load().natten_b200_merge_forward(_DTYPES[o0.dtype], rows, o0.shape[-1], _ptr(o0), _ptr(l0),
                                                         _ptr(o1), _ptr(l1), _ptr(out), _ptr(lse), _stream(o0)))
    return out, lse


def merge_backward(o0, l0, o1, l1, grad_out, grad_lse):
    o0, o1, grad_out = _prep(o0, o1, grad_out)
    l0, l1 = l0.to(torch.float32).contiguous(), l1.to(torch.float32).contiguous()
    if grad_lse is not None:
        grad_lse = grad_lse.to(torch.float32).contiguous()
    do0, do1 = torch.empty_like(o0), torch.empty_like(o1)
    dl0, dl1 = torch.empty_like(l0), torch.empty_like(l1)
    with torch.cuda.device(o0.device):
        _lib.check(_lib.load().natten_b200_merge_backward(
            _DTYPES[o0.dtype], l0.numel(), o0.shape[-1], _ptr(o0), _ptr(l0), _ptr(o1), _ptr(l1), _ptr(grad_out),
            _ptr(grad_lse), _ptr(do0), _ptr(dl0), _ptr(do1), _ptr(dl1), _stream(o0)))
    return do0, dl0, do1, dl1


# ---------------------------------------------------------------------------
# the backend-module protocol (names and argument order of the reference)
# ---------------------------------------------------------------------------

def _fwd(q, k, v, kernel_size, stride, dilation, is_causal, scale):
    return fused_forward(q, k, v, kernel_size, stride, dilation, is_causal, scale)[0]


def _bwd(q, k, v, grad_out, kernel_size, stride, dilation, is_causal, scale):
    out, lse = fused_forward(q, k, v, kernel_size, stride, dilation, is_causal, scale)
    return fused_backward(q, k, v, out, lse, grad_out, None, kernel_size, stride, dilation, is_causal, scale)[:3]


def _varlen_fwd(q, k, v, sizes, kernel_size, dilation, scale):
    rank = q.dim() - 3
    return fused_forward(q, k, v, kernel_size, (1,) * rank, dilation, (False,) * rank, scale, sizes=sizes)[0]


def _varlen_bwd(q, k, v, grad_out, sizes, kernel_size, dilation, scale):
    rank = q.dim() - 3
    one, no = (1,) * rank, (False,) * rank
    out, lse = fused_forward(q, k, v, kernel_size, one, dilation, no, scale, sizes=sizes)
    return fused_backward(q, k, v, out, lse, grad_out, None, kernel_size, one, dilation, no, scale, sizes=sizes)[:3]


na1d_forward = na2d_forward = na3d_forward = _fwd
na1d_backward = na2d_backward = na3d_backward = _bwd
na1d_qk_forward = na2d_qk_forward = na3d_qk_forward = lambda q, k, ks, st, dl, ca, scale: qk_forward(q, k, ks, st, dl, ca, scale)
na1d_qk_backward = na2d_qk_backward = na3d_qk_backward = lambda q, k, g, ks, st, dl, ca, scale: qk_backward(q, k, g, ks, st, dl, ca, scale)
na1d_av_forward = na2d_av_forward = na3d_av_forward = av_forward
na1d_av_backward = na2d_av_backward = na3d_av_backward = av_backward
na1d_varlen_forward = na2d_varlen_forward = na3d_varlen_forward = _varlen_fwd
na1d_varlen_backward = na2d_varlen_backward = na3d_varlen_backward = _varlen_bwd
