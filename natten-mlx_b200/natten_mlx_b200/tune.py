"""Measured tiling choice for the tensor-core kernels of one geometry.

The planner inside the library picks tile shape and chunk width from a cost
model.  ``tune_fused`` times a handful of alternatives on the caller's own
tensors (CUDA events, a few launches each) and records the fastest per kernel
through ``natten_b200_plan_hint``; later calls with the same geometry use it.
This plays the role of the reference's tuning tables
(``src/natten_mlx/_core/_forward_tuning.py:11-34``, ``_softmax_tuning.py``),
filled by measurement instead of by hand.  It synchronises the device: call it
once per shape, outside any stream capture.
"""

from __future__ import annotations

import ctypes
import itertools
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _lib
from ._core import cuda as backend
from .utils.params import normalize_kernel_size, normalize_tuple_param

_KERNELS = {0: "fna_fwd_sm100", 1: "fna_bwd_dq_sm100", 2: "fna_bwd_dkv_sm100"}


def _tile_shapes(rank: int, rows: int):
    """Power-of-two tile extents per axis whose product is the number of positions of a tile."""
    exps = [e for e in itertools.product(range(0, 8), repeat=rank) if sum(e) == rows.bit_length() - 1]
    return [tuple(1 << x for x in e) for e in exps]


def tune_fused(query, key, value, kernel_size, dilation=1, is_causal=False, scale: Optional[float] = None,
               max_cols: Sequence[int] = (0, 256, 192, 128, 96, 80, 64, 48), repeats: int = 3, verbose: bool = False,
               sizes=None, host_sizes=None, additional_keys=None, additional_values=None
               ) -> Dict[str, Tuple[Tuple[int, ...], int, float]]:
    """Times candidate tilings of the fused forward and backward for these tensors and pins the best.

    ``sizes`` / ``host_sizes`` (per-sample extents on the device and their host copy) and the extra tokens
    describe a variable-size call; the pinned tilings apply to calls of exactly that geometry.
    Returns ``{kernel name: (tile, max_cols, milliseconds)}`` of the winners.  Shapes the tensor-core
    kernels do not take are left alone (empty result)."""
    rank = query.dim() - 3
    ks = normalize_kernel_size(kernel_size, rank)
    dl = tuple(int(d) for d in normalize_tuple_param(dilation, rank, "dilation"))
    ca = tuple(bool(c) for c in normalize_tuple_param(is_causal, rank, "is_causal"))
    one = (1,) * rank
    if not query.is_cuda or query.dtype not in (torch.float16, torch.bfloat16):
        return {}
    sc = query.shape[-1] ** -0.5 if scale is None else float(scale)
    n_extra = 0 if additional_keys is None else int(additional_keys.shape[1])
    if sizes is not None:
        sizes = backend._sizes_tensor(sizes, query.shape[0], rank, query.device)
        host_sizes = backend._host_sizes(sizes, host_sizes, query.shape[0], rank)
    geom = _lib.make_geom(rank, query.shape[0], query.shape[-2], key.shape[-2], query.shape[-1],
                          {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}[query.dtype],
                          tuple(query.shape[1:1 + rank]), ks, one, dl, [int(c) for c in ca], sc, n_extra=n_extra,
                          extents_ptr=0 if sizes is None else sizes.data_ptr(),
                          host_extents=None if sizes is None else host_sizes)
    try:
        if "unsupported" in _lib.describe_plan(geom):
            return {}
    except ValueError:
        return {}
    lib = _lib.load()
    rep = query.shape[-2] // key.shape[-2]
    packed = 4 if rep % 4 == 0 else (2 if rep % 2 == 0 else 1)
    cot = torch.ones_like(query)

    def hint(kernel, tile, cols):
        arr = (ctypes.c_int32 * 3)(*(list(tile) + [0] * (3 - rank))) if tile is not None else None
        return lib.natten_b200_plan_hint(geom, kernel, arr, int(cols))

    def run_once():
        extra = dict(k_extra=additional_keys, v_extra=additional_values, sizes=sizes, host_sizes=host_sizes)
        out, lse = backend.fused_forward(query, key, value, ks, one, dl, ca, sc, path="tcgen05", **extra)
        backend.fused_backward(query, key, value, out, lse, cot, None, ks, one, dl, ca, sc, path="tcgen05", **extra)

    def measure():
        run_once()                                     # warm: attribute setting, plan building, caches
        torch.cuda.synchronize(query.device)
        _lib.trace_report()
        _lib.trace_enable(True)
        for _ in range(repeats):
            run_once()
        torch.cuda.synchronize(query.device)
        _lib.trace_enable(False)
        tr = _lib.trace_report()
        return {k: ms / n for k, (n, ms) in tr.items()}

    for kernel in _KERNELS:
        hint(kernel, None, 0)
    base = measure()
    best = {kernel: (None, 0, base.get(name, float("inf"))) for kernel, name in _KERNELS.items()}
    rows = {0: 128 // packed, 1: 128 // packed, 2: 128}
    # the planner's own tiles (first three numbers of each part of the description), as the centre of the search
    parts = _lib.describe_plan(geom).split(" | ")
    centre = {}
    for kernel in _KERNELS:
        dims = parts[kernel].split("tile ")[1].split(" ")[0].split("x")
        centre[kernel] = tuple(int(x) for x in dims)[3 - rank:]

    def near(tile, ref):                             # every axis within a factor of two of the planner's tile
        return all(t in (r // 2, r, r * 2) for t, r in zip(tile, ref))
    # the kernels are independent of each other: one candidate per kernel is timed in the same pass
    cands = {kernel: [(t, c) for t in _tile_shapes(rank, rows[kernel]) if near(t, centre[kernel]) for c in max_cols]
             for kernel in _KERNELS}
    width = max(len(v) for v in cands.values())
    for i in range(width):
        active = {}
        for kernel, lst in cands.items():
            if i < len(lst) and hint(kernel, lst[i][0], lst[i][1]) == _lib.OK:
                active[kernel] = lst[i]
            else:
                hint(kernel, best[kernel][0], best[kernel][1])
        if not active:
            continue
        times = measure()
        for kernel, (tile, cols) in active.items():
            t = times.get(_KERNELS[kernel], float("inf"))
            if verbose:
                print(f"{_KERNELS[kernel]} tile {tile} max_cols {cols}: {t * 1e3:.1f} us")
            if t < best[kernel][2] * 0.98:             # keep the planner's choice unless clearly beaten
                best[kernel] = (tile, cols, t)
    result = {}
    for kernel, (tile, cols, t) in best.items():
        hint(kernel, tile, cols)
        result[_KERNELS[kernel]] = (tile if tile is not None else (), cols, t)
    if int(lib.natten_b200_kernel_status()) != 0:
        raise _lib.NattenB200Error("a tensor-core kernel gave up on a wait while tuning")
    return result


__all__ = ["tune_fused"]
