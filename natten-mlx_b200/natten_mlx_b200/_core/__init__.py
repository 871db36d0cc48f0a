"""Backend layer: the dispatcher and its single ``cuda`` backend."""
