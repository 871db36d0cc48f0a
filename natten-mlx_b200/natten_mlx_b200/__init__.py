"""Neighborhood attention for NVIDIA B200: the operator surface of natten-mlx
(src/natten_mlx/__init__.py:15-36) on torch CUDA tensors, backed by one
``cuda`` backend made of hand-written sm_100a kernels behind a C ABI."""

from __future__ import annotations

from ._core import ops
from ._core.cuda import get_fused_path, set_fused_path
from .functional import (na1d, na1d_av, na1d_qk, na1d_varlen, na2d, na2d_av, na2d_qk, na2d_varlen, na3d,
                         na3d_av, na3d_qk, na3d_varlen)
from .merge import merge_attentions
from . import compat, host, nn, tune  # noqa: E402  (callers of the operators: modules, old call conventions, host-resident tensors)

__version__ = "0.1.0"


def has_cuda() -> bool:
    """True when the compiled library loads and a CUDA device is visible."""
    return ops._BACKEND_REGISTRY["cuda"].is_available()


def get_backend() -> str:
    return ops.get_backend()


def set_backend(name: str) -> None:
    ops.set_backend(name)


__all__ = [
    "__version__", "get_backend", "set_backend", "has_cuda", "get_fused_path", "set_fused_path",
    "merge_attentions", "nn", "compat", "host", "tune",
    "na1d", "na1d_av", "na1d_qk", "na1d_varlen",
    "na2d", "na2d_av", "na2d_qk", "na2d_varlen",
    "na3d", "na3d_av", "na3d_qk", "na3d_varlen",
]
