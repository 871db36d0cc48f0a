"""A torch-backed stand-in for the few ``mlx.core`` calls the reference's CPU path makes.

Used ONLY by ``make_golden.py`` (fixture generation, run where the reference
sources are present).  The reference's pure backend is Python over the MLX
array library, which cannot be installed on Linux without a network.  Its own
code (window tables, gathers, masking, softmax composition, autodiff-defined
backward, LSE / extra-token / merge composition, allin1 QK+RPB) is executed
unmodified; only the array primitives underneath are supplied here by torch on
the CPU.  Nothing in the product or in the tests imports this file.
"""

from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch


def _install_tensor_methods():
    if not hasattr(torch.Tensor, "astype"):
        torch.Tensor.astype = lambda self, dt: self.to(dt)


def _as_tensor(x, dtype=None):
    if torch.is_tensor(x):
        return x if dtype is None else x.to(dtype)
    if isinstance(x, (bool, int, float)):
        t = torch.tensor(x)
        if isinstance(x, float) and dtype is None:
            t = t.float()
        return t if dtype is None else t.to(dtype)
    t = torch.from_numpy(np.ascontiguousarray(np.asarray(x)))
    if t.dtype == torch.float64 and dtype is None:
        t = t.float()
    return t if dtype is None else t.to(dtype)


def _take(x, idx, axis=None):
    idx = _as_tensor(idx).long()
    if axis is None:
        return x.reshape(-1)[idx]
    return torch.index_select(x, axis, idx.reshape(-1))


def _grad(fn):
    def run(x):
        leaf = x.detach().clone().requires_grad_(True)
        with torch.enable_grad():
            y = fn(leaf)
        return torch.autograd.grad(y, leaf)[0]
    return run


def _pad(x, pad_width, constant_values=0):
    flat = []
    for lo, hi in reversed(list(pad_width)):
        flat += [int(lo), int(hi)]
    return torch.nn.functional.pad(x, flat, value=constant_values)


def _sdpa(q, k, v, scale=None, mask=None):
    s = (q @ k.transpose(-1, -2)) * (q.shape[-1] ** -0.5 if scale is None else scale)
    return torch.softmax(s, dim=-1) @ v


def build_modules():
    _install_tensor_methods()
    core = types.ModuleType("mlx.core")
    core.array = _as_tensor
    for name in ("int32", "int64", "float32", "float16", "bfloat16", "float64"):
        setattr(core, name, getattr(torch, name))
    core.bool_ = torch.bool
    core.inf = float("inf")
    core.take = _take
    core.reshape = lambda x, shape: x.reshape(tuple(shape))
    core.transpose = lambda x, axes=None: x.permute(*axes) if axes is not None else x.T
    core.sum = lambda x, axis=None, keepdims=False: x.sum() if axis is None else x.sum(dim=axis, keepdim=keepdims)
    core.where = lambda c, a, b: torch.where(c, a if torch.is_tensor(a) else torch.tensor(a, dtype=(b.dtype if torch.is_tensor(b) else torch.float32)),
                                              b if torch.is_tensor(b) else torch.tensor(b, dtype=(a.dtype if torch.is_tensor(a) else torch.float32)))
    core.softmax = lambda x, axis=-1: torch.softmax(x, dim=axis)
    core.logsumexp = lambda x, axis=-1: torch.logsumexp(x, dim=axis)
    core.full = lambda shape, val, dtype=None: torch.full(tuple(shape), val, dtype=dtype or torch.float32)
    core.zeros = lambda shape, dtype=None: torch.zeros(tuple(shape), dtype=dtype or torch.float32)
    core.concatenate = lambda xs, axis=0: torch.cat(list(xs), dim=axis)
    core.stack = lambda xs, axis=0: torch.stack(list(xs), dim=axis)
    core.eval = lambda *a, **k: None
    core.grad = _grad
    core.clip = lambda x, lo, hi: torch.clamp(x, lo, hi)
    core.min = lambda x, axis=None: x.min() if axis is None else x.min(dim=axis).values
    core.max = lambda x, axis=None: x.max() if axis is None else x.max(dim=axis).values
    core.pad = _pad
    core.sigmoid = torch.sigmoid
    core.squeeze = lambda x, axis=None: x.squeeze() if axis is None else x.squeeze(axis)
    core.expand_dims = lambda x, axis: x.unsqueeze(axis)
    core.repeat = lambda x, n, axis=None: torch.repeat_interleave(x, n, dim=axis)
    fast = types.ModuleType("mlx.core.fast")
    fast.scaled_dot_product_attention = _sdpa
    core.fast = fast

    nn = types.ModuleType("mlx.nn")
    nn.log_sigmoid = torch.nn.functional.logsigmoid

    top = types.ModuleType("mlx")
    top.core = core
    top.nn = nn
    return {"mlx": top, "mlx.core": core, "mlx.core.fast": fast, "mlx.nn": nn}


def load_reference(src_root: str):
    """Import the reference's CPU path from ``src_root`` (its ``src`` folder).

    The package's ``__init__`` refuses to import off macOS, and its accelerated
    tiers need Metal; both are bypassed by registering empty package shells and
    two unavailable-tier placeholders, then importing the real modules below.
    Returns a namespace with the modules that matter.
    """
    os.environ["NATTEN_BACKEND"] = "pure"
    sys.modules.update(build_modules())
    pkg_dir = os.path.join(src_root, "natten_mlx")

    def shell(name, path):
        m = types.ModuleType(name)
        m.__path__ = [path]
        sys.modules[name] = m
        return m

    shell("natten_mlx", pkg_dir)
    shell("natten_mlx._core", os.path.join(pkg_dir, "_core"))
    shell("natten_mlx.extras", os.path.join(pkg_dir, "extras"))
    for tier in ("fast_metal", "nanobind"):
        m = types.ModuleType(f"natten_mlx._core.{tier}")
        m.is_available = lambda: False
        sys.modules[f"natten_mlx._core.{tier}"] = m
        setattr(sys.modules["natten_mlx._core"], tier, m)

    import importlib
    ns = types.SimpleNamespace()
    ns.window = importlib.import_module("natten_mlx.utils.window")
    ns.pure = importlib.import_module("natten_mlx._core.pure")
    setattr(sys.modules["natten_mlx._core"], "pure", ns.pure)
    ns.ops = importlib.import_module("natten_mlx._core.ops")
    ns.ops.register_backend("pure", ns.pure)
    ns.functional = importlib.import_module("natten_mlx.functional")
    ns.merge = importlib.import_module("natten_mlx.merge")
    ns.allin1_ref = importlib.import_module("natten_mlx.extras.allin1.reference_impl")
    ns.allin1 = importlib.import_module("natten_mlx.extras.allin1")
    # The Metal tier of allin1 imports but cannot run here; select its own
    # pure fallback branch (extras/allin1/__init__.py:74-79).
    for name in ("_metal_1d_qkrpb", "_metal_1d_av", "_metal_2d_qkrpb", "_metal_2d_av"):
        setattr(ns.allin1, name, None)
    return ns
