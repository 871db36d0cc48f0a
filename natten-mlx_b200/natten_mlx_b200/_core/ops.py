"""Backend dispatch (the interface of src/natten_mlx/_core/ops.py:10-143).

The registry holds one backend, ``cuda``; ``auto`` resolves to it.  A call
never falls back to another implementation: when the backend cannot run
(no library, no GPU) the call raises.
"""

from __future__ import annotations

import os
from typing import Any

from . import cuda

_BACKEND_REGISTRY: dict[str, Any] = {}
_ACTIVE_BACKEND = os.environ.get("NATTEN_BACKEND", "auto")
_VALID = ("auto", "cuda")


def register_backend(name: str, module: Any) -> None:
    _BACKEND_REGISTRY[name] = module


def _resolve_backend() -> str:
    return "cuda" if _ACTIVE_BACKEND == "auto" else _ACTIVE_BACKEND


def get_backend() -> str:
    return _resolve_backend()


def set_backend(name: str) -> None:
    global _ACTIVE_BACKEND
    if name not in _VALID:
        raise ValueError(f"Unknown backend {name!r}. Expected one of {sorted(_VALID)}")
    _ACTIVE_BACKEND = name


def _backend_module() -> Any:
    name = _resolve_backend()
    try:
        return _BACKEND_REGISTRY[name]
    except KeyError as exc:
        raise RuntimeError(f"Backend {name!r} is not registered") from exc


def _forwarder(fn_name: str):
    def call(*args, **kwargs):
        return getattr(_backend_module(), fn_name)(*args, **kwargs)
    call.__name__ = fn_name
    call.__doc__ = f"Dispatch ``{fn_name}`` to the active backend."
    return call


for _rank in (1, 2, 3):
    for _op in ("forward", "backward", "qk_forward", "qk_backward", "av_forward", "av_backward",
                "varlen_forward", "varlen_backward"):
        _name = f"na{_rank}d_{_op}"
        globals()[_name] = _forwarder(_name)

register_backend("cuda", cuda)
