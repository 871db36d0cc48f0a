"""Window helpers with the signatures of src/natten_mlx/utils/window.py:8-103.

The integers come from the library's host-side table routine, i.e. from the
same code the kernels execute; it needs no GPU.
"""

from __future__ import annotations

import ctypes

import numpy as np

from .. import _lib


def _table(length: int, kernel_size: int, dilation: int, stride: int, causal: bool):
    n = -(-length // stride)
    idx = np.empty((n, kernel_size), dtype=np.int32)
    valid = np.empty((n, kernel_size), dtype=np.uint8)
    start = np.empty((n,), dtype=np.int32)
    pb = np.empty((n,), dtype=np.int32)
    as_ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    rc = _lib.load().natten_b200_axis_table(length, kernel_size, dilation, stride, int(causal),
                                            as_ptr(idx), as_ptr(valid), as_ptr(start), as_ptr(pb))
    _lib.check(rc)
    return idx, valid.astype(bool), start, pb


def axis_table(length: int, kernel_size: int, dilation: int = 1, stride: int = 1, causal: bool = False):
    """(neighbour index clipped to the axis, validity, window start, bias start) per strided query."""
    return _table(int(length), int(kernel_size), int(dilation), int(stride), bool(causal))


def _starts(length: int, kernel_size: int, dilation: int) -> np.ndarray:
    return _table(length, kernel_size, dilation, 1, False)[2]


def get_window_start(index: int, length: int, kernel_size: int, neighborhood_size: int, dilation: int) -> int:
    return int(_starts(length, kernel_size, max(1, dilation))[index])


def get_window_end(start_index: int, length: int, kernel_size: int, dilation: int) -> int:
    return min(length, start_index + kernel_size * dilation)


def get_pb_start(index: int, length: int, kernel_size: int, neighborhood_size: int, dilation: int) -> int:
    return int(_table(length, kernel_size, max(1, dilation), 1, False)[3][index])


def compute_window_start_end(query_positions, length: int, kernel_size: int, dilation: int):
    pos = np.asarray(query_positions, dtype=np.int64)
    starts = _starts(length, kernel_size, max(1, dilation))[pos]
    ends = np.minimum(length, starts + kernel_size * dilation).astype(np.int32)
    return starts.astype(np.int32), ends


def compute_pb_start(query_positions, length: int, kernel_size: int, dilation: int) -> np.ndarray:
    pos = np.asarray(query_positions, dtype=np.int64)
    return _table(length, kernel_size, max(1, dilation), 1, False)[3][pos].astype(np.int32)
