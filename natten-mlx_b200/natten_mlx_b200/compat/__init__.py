"""Call conventions of historical NATTEN releases on top of the current operators
(the reference's selector: ``src/natten_mlx/compat/__init__.py:9-22``).

Only the v0.14 surface has a calling convention of its own (heads-first tensors, un-scaled
QK with a relative-position-bias table); later surfaces are the current functions."""

from __future__ import annotations

from importlib import import_module


def for_version(version: str):
    """Module that speaks the API of the given NATTEN release (``"0.14.6"``, ``"0.17"`` ...)."""
    parts = (str(version).split(".") + ["0"])[:2]
    try:
        target = (int(parts[0]), int(parts[1]))
    except ValueError as exc:
        raise ValueError(f"not a version string: {version!r}") from exc
    if target <= (0, 14):
        return import_module(__name__ + ".v014")
    return import_module(__name__.rsplit(".", 1)[0])


__all__ = ["for_version"]
