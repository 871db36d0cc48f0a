"""Host-side checks that need no GPU: the shared library loads, exports every
symbol the header declares, evaluates the integer window tables bit-exactly and
rejects bad geometry before touching CUDA; the Python API raises the
reference's ``ValueError``s."""

from __future__ import annotations

import ctypes
import os
import re

import numpy as np
import pytest
import torch

from conftest import GOLDEN, ROOT
from make_golden import window_grid

import natten_mlx_b200 as nb
from natten_mlx_b200 import _lib
from natten_mlx_b200.utils import window as W


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "natten_b200.h")).read()
    declared = set(re.findall(r"\b(natten_b200_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 14
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_lib.SYMBOLS), "ctypes table and header disagree"
    assert _lib.load().natten_b200_abi_version() == 2


def test_geom_struct_layout_matches_header():
    # the C side pins the same numbers with static_assert (csrc/api.cu)
    assert ctypes.sizeof(_lib.Geom) == 176
    assert _lib.Geom.extents.offset == 144 and _lib.Geom.scale.offset == 132 and _lib.Geom.host_extents.offset == 168


def test_axis_table_matches_reference_tables_bit_exact():
    t = np.load(os.path.join(GOLDEN, "window_tables.npz"))
    for (length, k, d), off in zip(t["grid"], t["offsets"]):
        length, k, d = int(length), int(k), int(d)
        idx, valid, start, pb = W.axis_table(length, k, d)
        assert start.tolist() == t["starts"][off:off + length].tolist(), (length, k, d)
        assert pb.tolist() == t["pb_starts"][off:off + length].tolist(), (length, k, d)
        ends = np.minimum(length, start + k * d)
        assert ends.tolist() == t["ends"][off:off + length].tolist()
        raw = start[:, None] + np.arange(k)[None, :] * d
        assert np.array_equal(valid, (raw >= 0) & (raw < ends[:, None]))
        assert np.array_equal(idx, np.clip(raw, 0, length - 1))


def test_axis_table_matches_reference_index_tables():
    t = np.load(os.path.join(GOLDEN, "index_tables.npz"))
    off = 0
    for length, k, d, stride, causal, n in t["axis_cases"]:
        idx, valid, _, _ = W.axis_table(int(length), int(k), int(d), int(stride), bool(causal))
        m = int(n) * int(k)
        assert idx.reshape(-1).tolist() == t["axis_idx"][off:off + m].tolist()
        assert valid.reshape(-1).tolist() == t["axis_ok"][off:off + m].tolist()
        off += m


def test_window_helpers_known_answers():
    # tests/test_shift_semantics.py:53-64 of the reference
    assert W.get_window_start(31, 32, 3, 1, 1) == 29
    assert W.get_pb_start(31, 32, 3, 1, 1) == 0
    s, e = W.compute_window_start_end(np.arange(10), 10, 3, 2)
    assert (s % 2 == np.arange(10) % 2).all() and (e <= 10).all()


def _geom(**kw):
    base = dict(rank=1, batch=1, heads_q=2, heads_kv=2, head_dim=8, dtype=_lib.F32, extent=[16], kernel=[3],
                stride=[1], dilation=[1], causal=[0], scale=1.0)
    base.update(kw)
    return _lib.make_geom(**base)


@pytest.mark.parametrize("kw,needle", [
    (dict(rank=0), "rank"), (dict(kernel=[0]), "kernel_size"), (dict(kernel=[17]), "kernel_size"),
    (dict(stride=[4]), "stride"), (dict(kernel=[5], dilation=[4]), "dilation"),
    (dict(heads_q=3), "divisible"), (dict(dtype=7), "dtype"),
    (dict(q_extent=[8], q_offset=[4], kv_extent=[8], kv_offset=[4]), "local key slab"),
])
def test_bad_geometry_is_rejected_without_a_gpu(kw, needle):
    lib = _lib.load()
    rc = lib.natten_b200_qk_forward(_geom(**kw), 8, 8, None, 8, None)   # never dereferenced
    assert rc == _lib.EINVAL
    assert needle in _lib.last_error()
    with pytest.raises(ValueError):
        _lib.check(rc)


def test_null_pointers_are_rejected():
    lib = _lib.load()
    assert lib.natten_b200_fused_forward(_geom(), None, None, None, None, None, None, None, None) == _lib.EINVAL
    assert lib.natten_b200_av_forward(_geom(), None, None, None, None) == _lib.EINVAL
    assert lib.natten_b200_merge_forward(0, 4, 8, None, None, None, None, None, None, None) == _lib.EINVAL
    assert lib.natten_b200_fused_backward_scratch_bytes(_geom()) >= 16 * 2 * 4


def test_misaligned_pointers_are_rejected_before_any_launch():
    """Rows travel through 16-byte vector accesses and TMA maps: a base address that is not a multiple
    of 16 is refused with EINVAL on the host (nothing is dereferenced or launched)."""
    lib = _lib.load()
    before = _lib.launch_count()
    assert lib.natten_b200_qk_forward(_geom(), 4096 + 8, 4096, None, 4096, None) == _lib.EINVAL
    assert "16-byte aligned" in _lib.last_error()
    assert lib.natten_b200_av_forward(_geom(), 4096, 4096 + 2, 4096, None) == _lib.EINVAL
    assert lib.natten_b200_fused_forward(_geom(), 4096, 4096, 4096 + 4, None, None, 4096, None, None) == _lib.EINVAL
    assert lib.natten_b200_fused_backward(_geom(), 4096, 4096, 4096, None, None, 4096, 4096, 4096, None, 4096, 4096 + 12,
                                          4096, None, None, 4096, 1 << 20, None) == _lib.EINVAL
    assert lib.natten_b200_merge_forward(0, 4, 8, 4096 + 1, 4096, 4096, 4096, 4096, 4096, None) == _lib.EINVAL
    assert _lib.launch_count() == before


def test_backend_registry():
    assert nb.get_backend() == "cuda"
    with pytest.raises(ValueError):
        nb.set_backend("pure")
    nb.set_backend("auto")
    assert nb.get_backend() == "cuda"
    with pytest.raises(ValueError):
        nb.set_fused_path("metal")


def test_no_cpu_path():
    q = torch.randn(1, 16, 2, 8)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        nb.na1d(q, q, q, kernel_size=3)


# ---- ValueErrors of the public API (texts matched by the reference's tests) ------------

def test_validation_errors():
    q = torch.randn(1, 16, 2, 8)
    with pytest.raises(ValueError, match="na1d"):
        nb.na1d(q[0], q[0], q[0], kernel_size=3)
    with pytest.raises(ValueError, match="na2d"):
        nb.na2d(q, q, q, kernel_size=3)
    with pytest.raises(ValueError, match="Spatial dimensions must match"):
        nb.na1d(q, q[:, :8], q[:, :8], kernel_size=3)
    with pytest.raises(ValueError, match="Head dim must match"):
        nb.na1d(q, q[..., :4], q[..., :4], kernel_size=3)
    with pytest.raises(ValueError, match="divisible"):
        nb.na1d(torch.randn(1, 16, 3, 8), q, q, kernel_size=3)
    with pytest.raises(ValueError, match="both be provided"):
        nb.na1d(q, q, q, kernel_size=3, additional_keys=torch.randn(1, 2, 2, 8))
    with pytest.raises(ValueError, match="batch"):
        nb.na1d(q, q, q, kernel_size=3, additional_keys=torch.randn(2, 2, 2, 8), additional_values=torch.randn(2, 2, 2, 8))
    with pytest.raises(ValueError, match="head dim"):
        nb.na1d(q, q, q, kernel_size=3, additional_keys=torch.randn(1, 2, 2, 4), additional_values=torch.randn(1, 2, 2, 4))
    with pytest.raises(ValueError, match="kernel_size"):
        nb.na1d(q, q, q, kernel_size=17)
    with pytest.raises(ValueError, match="stride"):
        nb.na1d(q, q, q, kernel_size=3, stride=4)
    with pytest.raises(ValueError, match="exceeds input size"):
        nb.na1d(q, q, q, kernel_size=5, dilation=4)
    with pytest.raises(ValueError, match="length 2"):
        nb.na2d(torch.randn(1, 8, 8, 2, 4), torch.randn(1, 8, 8, 2, 4), torch.randn(1, 8, 8, 2, 4), kernel_size=(3, 3, 3))
    with pytest.raises(ValueError, match="at least two"):
        nb.merge_attentions([q], [q[..., 0]])
    with pytest.raises(ValueError, match="must match"):
        nb.merge_attentions([q, q], [q[..., 0]])
    with pytest.raises(ValueError, match="shape"):
        nb.merge_attentions([q, q[:, :8]], [q[..., 0], q[:, :8, :, 0]])
    with pytest.raises(ValueError, match="kernel_size"):
        nb.na1d_varlen(q, q, q, torch.tensor([2], dtype=torch.int32), kernel_size=3)
    with pytest.raises(ValueError, match="L_max"):
        nb.na1d_varlen(q, q, q, torch.tensor([20], dtype=torch.int32), kernel_size=3)
    with pytest.raises(ValueError, match="int32 or int64"):
        nb.na1d_varlen(q, q, q, torch.tensor([8.0]), kernel_size=3)
    q2 = torch.randn(1, 8, 8, 2, 4)
    with pytest.raises(ValueError, match="max_spatial"):
        nb.na2d_varlen(q2, q2, q2, torch.tensor([[9, 8]], dtype=torch.int32), kernel_size=3)
    from natten_mlx_b200.extras import allin1
    with pytest.raises(ValueError, match="4D"):
        allin1.na1d_qk_rpb(q2, q2, None, 3)
    with pytest.raises(ValueError, match="5D"):
        allin1.na2d_qk_rpb(q, q, None, 3)
    with pytest.raises(ValueError, match="kernel volume|kernel area|neighborhood dimension"):
        from natten_mlx_b200._core import cuda
        cuda._check_attn(torch.randn(1, 16, 2, 4), q, 1, (3,), (1,))


def test_planner_is_host_only_and_breaks_ties_by_needed_rows():
    """The tiling plan is worked out on the host (no GPU needed to describe it).  At dilation 4 a
    56x56 image has 14x14 positions per dilation class: a 16x8 and an 8x16 key tile cost the same
    padded columns, but the queries that address an 8-row key tile span fewer box rows, and the
    elementwise warps skip the rows nobody needs, so the planner takes 8x16 for dK/dV."""
    g = _lib.make_geom(2, 32, 4, 4, 32, _lib.BF16, (56, 56), (7, 7), (1, 1), (4, 4), [0, 0], 32 ** -0.5)
    parts = _lib.describe_plan(g).split(" | ")
    assert len(parts) == 3 and all("unsupported" not in p for p in parts)
    assert "tile 1x8x16" in parts[2] and "box 1x14x16" in parts[2]
    # dilation 1: the key box of a 16x8 query tile is 22 rows of 14 -> 16 padded columns
    g1 = _lib.make_geom(2, 32, 4, 4, 32, _lib.BF16, (56, 56), (7, 7), (1, 1), (1, 1), [0, 0], 32 ** -0.5)
    fwd = _lib.describe_plan(g1).split(" | ")[0]
    assert "tile 1x16x8" in fwd and "box 1x22x16" in fwd and "2 CTA/SM" in fwd
    # a shape the tensor-core kernels do not take says why
    gbad = _lib.make_geom(1, 4, 8, 8, 64, _lib.BF16, (8192,), (127,), (1,), (1,), [0], 64 ** -0.5)
    assert "unsupported" in _lib.describe_plan(gbad)
