"""ctypes binding of ``libnatten_b200.so`` (the C ABI declared in ``include/natten_b200.h``).

The library is the only compute path: if it is missing or a symbol cannot be
resolved the import of a compute entry point raises; nothing falls back to
another implementation.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnatten_b200.so")

F32, F16, BF16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TCGEN05 = 0, 1, 2

OK, EINVAL, ELAUNCH, ERESOURCE, ENODEVICE = 0, 1, 2, 3, 4

_I3 = ctypes.c_int32 * 3


class Geom(ctypes.Structure):
    """Mirror of ``natten_b200_geom``."""

    _fields_ = [
        ("rank", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("heads_q", ctypes.c_int32),
        ("heads_kv", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("q_extent", _I3),
        ("kv_extent", _I3),
        ("global_extent", _I3),
        ("q_offset", _I3),
        ("kv_offset", _I3),
        ("kernel", _I3),
        ("stride", _I3),
        ("dilation", _I3),
        ("causal", _I3),
        ("scale", ctypes.c_float),
        ("n_extra", ctypes.c_int32),
        ("path", ctypes.c_int32),
        ("extents", ctypes.c_void_p),
        ("mem_extent", _I3),
        ("reserved", ctypes.c_int32),
        ("host_extents", ctypes.c_void_p),
    ]


_P = ctypes.c_void_p
_G = ctypes.POINTER(Geom)

# name -> (restype, argtypes); every symbol the header declares.
SYMBOLS = {
    "natten_b200_abi_version": (ctypes.c_int, []),
    "natten_b200_last_error": (ctypes.c_char_p, []),
    "natten_b200_last_path": (ctypes.c_char_p, []),
    "natten_b200_launch_count": (ctypes.c_uint64, []),
    "natten_b200_trace_enable": (None, [ctypes.c_int]),
    "natten_b200_trace_report": (ctypes.c_size_t, [ctypes.c_char_p, ctypes.c_size_t]),
    "natten_b200_axis_table": (ctypes.c_int, [ctypes.c_int32] * 5 + [_P, _P, _P, _P]),
    "natten_b200_qk_forward": (ctypes.c_int, [_G, _P, _P, _P, _P, _P]),
    "natten_b200_qk_backward": (ctypes.c_int, [_G, _P, _P, _P, _P, _P, _P, _P]),
    "natten_b200_av_forward": (ctypes.c_int, [_G, _P, _P, _P, _P]),
    "natten_b200_qk_bias_av_forward": (ctypes.c_int, [_G, _P, _P, _P, _P, _P, _P, _P]),
    "natten_b200_av_backward": (ctypes.c_int, [_G, _P, _P, _P, _P, _P, _P]),
    "natten_b200_fused_forward": (ctypes.c_int, [_G] + [_P] * 8),
    "natten_b200_fused_backward_scratch_bytes": (ctypes.c_size_t, [_G]),
    "natten_b200_fused_backward": (ctypes.c_int, [_G] + [_P] * 15 + [ctypes.c_size_t, _P]),
    "natten_b200_static_scratch_capacity": (ctypes.c_size_t, []),
    "natten_b200_fused_backward_static_scratch": (ctypes.c_int, [_G] + [_P] * 15),
    "natten_b200_fused_backward_halo": (ctypes.c_int, [_G] + [_P] * 11 + [ctypes.c_size_t, _P, _P]),
    "natten_b200_kernel_status": (ctypes.c_int, []),
    "natten_b200_peer_copy2d": (ctypes.c_int, [_P, ctypes.c_size_t, _P, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, _P]),
    "natten_b200_peer_copy2d_dma": (ctypes.c_int, [_P, ctypes.c_size_t, _P, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, _P]),
    "natten_b200_peer_barrier": (ctypes.c_int, [_P, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint32, ctypes.c_uint32, _P]),
    "natten_b200_describe_plan": (ctypes.c_int, [_G, ctypes.c_char_p, ctypes.c_size_t]),
    "natten_b200_plan_hint": (ctypes.c_int, [_G, ctypes.c_int32, _P, ctypes.c_int32]),
    "natten_b200_merge_forward": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int64, ctypes.c_int32] + [_P] * 7),
    "natten_b200_merge_backward": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int64, ctypes.c_int32] + [_P] * 11),
}

class HaloOut(ctypes.Structure):
    """Mirrors natten_b200_halo_out: where the dK / dV of a slab's halo planes go."""
    _fields_ = [("planes_below", ctypes.c_int32), ("planes_above", ctypes.c_int32),
                ("dk_below", ctypes.c_void_p), ("dv_below", ctypes.c_void_p),
                ("dk_above", ctypes.c_void_p), ("dv_above", ctypes.c_void_p)]


_lib: Optional[ctypes.CDLL] = None


class NattenB200Error(RuntimeError):
    """A launch- or resource-level failure reported by the library."""


def load() -> ctypes.CDLL:
    """Load the shared library once and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python natten-mlx_b200/build.py` "
            "(the package has no other compute path)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.natten_b200_abi_version() != 2:
        raise ImportError("libnatten_b200.so has an unexpected ABI version")
    _lib = lib
    return lib


def last_error() -> str:
    return load().natten_b200_last_error().decode()


def last_path() -> str:
    return load().natten_b200_last_path().decode()


def launch_count() -> int:
    return int(load().natten_b200_launch_count())


def trace_enable(on: bool) -> None:
    """Switch per-kernel CUDA-event timing inside the library on or off."""
    load().natten_b200_trace_enable(1 if on else 0)


def trace_report() -> dict:
    """{kernel name: (launches, total device ms)} since the last report; waits for the launches."""
    buf = ctypes.create_string_buffer(1 << 16)
    load().natten_b200_trace_report(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        out[name] = (int(n), float(ms))
    return out


def kernel_status() -> int:
    """Non-zero if a kernel gave up on a bounded wait since the last call (1 a tensor-core kernel, 2 a peer
    barrier); synchronises with the device."""
    return int(load().natten_b200_kernel_status())


def describe_plan(geom: "Geom") -> str:
    buf = ctypes.create_string_buffer(2048)
    check(load().natten_b200_describe_plan(geom, buf, len(buf)))
    return buf.value.decode()


def check(rc: int) -> None:
    """Map a status code to the exception the reference's API would raise."""
    if rc == OK:
        return
    msg = last_error()
    if rc == EINVAL:
        raise ValueError(msg)
    raise NattenB200Error(f"natten_b200 error {rc}: {msg}")


def make_geom(rank: int, batch: int, heads_q: int, heads_kv: int, head_dim: int, dtype: int,
              extent: Sequence[int], kernel: Sequence[int], stride: Sequence[int],
              dilation: Sequence[int], causal: Sequence[bool], scale: float, *,
              n_extra: int = 0, path: int = PATH_AUTO, extents_ptr: int = 0,
              q_extent: Optional[Sequence[int]] = None, kv_extent: Optional[Sequence[int]] = None,
              q_offset: Optional[Sequence[int]] = None, kv_offset: Optional[Sequence[int]] = None,
              mem_extent: Optional[Sequence[int]] = None, host_extents: Optional[Sequence[Sequence[int]]] = None) -> Geom:
    def arr(v, fill=0):
        v = list(v) + [fill] * (3 - len(v))
        return _I3(*[int(x) for x in v])

    g = Geom()
    g.rank, g.batch, g.heads_q, g.heads_kv, g.head_dim, g.dtype = rank, batch, heads_q, heads_kv, head_dim, dtype
    g.global_extent = arr(extent, 1)
    g.q_extent = arr(q_extent if q_extent is not None else extent, 1)
    g.kv_extent = arr(kv_extent if kv_extent is not None else extent, 1)
    g.q_offset = arr(q_offset if q_offset is not None else [0] * rank)
    g.kv_offset = arr(kv_offset if kv_offset is not None else [0] * rank)
    g.kernel, g.stride, g.dilation = arr(kernel, 1), arr(stride, 1), arr(dilation, 1)
    g.causal = arr([int(c) for c in causal])
    g.scale = float(scale)
    g.n_extra = int(n_extra)
    g.path = int(path)
    g.extents = extents_ptr or None
    g.mem_extent = arr(mem_extent if mem_extent is not None else [0] * rank)
    g.reserved = 0
    g.host_extents = None
    if host_extents is not None:
        flat = [int(x) for row in host_extents for x in (row if isinstance(row, (list, tuple)) else (row,))]
        arr_t = (ctypes.c_int32 * len(flat))(*flat)
        g._host_extents_keepalive = arr_t            # the struct only holds the address
        g.host_extents = ctypes.cast(arr_t, ctypes.c_void_p).value
    return g
