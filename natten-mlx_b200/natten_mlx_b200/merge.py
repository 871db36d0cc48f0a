"""``merge_attentions``: combine attention results that share queries as if
their key/value sets had been concatenated (src/natten_mlx/merge.py:20-68).

Each pairwise step is one CUDA kernel (float32 arithmetic, output in the input
dtype, LSE in float32) with its own backward; more than two inputs fold left
exactly as the reference does.
"""

from __future__ import annotations

from typing import List, Tuple

import torch

from . import autograd as _ag


def merge_attentions(outputs: List[torch.Tensor], lse_tensors: List[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """outputs: ``[B, ..spatial.., H, D]`` each; lse_tensors: ``[B, ..spatial.., H]`` each.
    Returns ``(merged_output, merged_lse)``."""
    if len(outputs) < 2:
        raise ValueError("merge_attentions expects at least two outputs.")
    if len(outputs) != len(lse_tensors):
        raise ValueError("Number of outputs and LSE tensors must match.")
    ref_shape = tuple(outputs[0].shape)
    for i, (o, l) in enumerate(zip(outputs, lse_tensors)):
        if tuple(o.shape) != ref_shape:
            raise ValueError(f"Output {i} shape {tuple(o.shape)} does not match output 0 shape {ref_shape}.")
        if tuple(l.shape) != ref_shape[:-1]:
            raise ValueError(f"LSE {i} shape {tuple(l.shape)} does not match expected {ref_shape[:-1]}.")
    out, lse = _ag.merge_pair_with_grad(outputs[0], lse_tensors[0].float(), outputs[1], lse_tensors[1].float())
    for i in range(2, len(outputs)):
        out, lse = _ag.merge_pair_with_grad(out, lse, outputs[i], lse_tensors[i].float())
    return out, lse


__all__ = ["merge_attentions"]
