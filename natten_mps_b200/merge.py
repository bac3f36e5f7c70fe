"""Merge attention outputs that share a query, as if their key/value sets had
been concatenated.

Given partial results ``(out_i, lse_i)`` the exact combination is
``lse = logsumexp_i(lse_i)`` and ``out = sum_i exp(lse_i - lse) * out_i``.
Accumulation is in float32 (float64 for float64 inputs); the output keeps the
dtype of ``outputs[0]`` and the merged lse is returned in the accumulation
dtype.  Same contract as the reference's ``src/natten_mps/merge.py:105-156``;
the fused kernels fold additional tokens into one softmax directly, so this
function is for user code that merges separately computed attentions.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
from torch import Tensor


def merge_attentions(outputs: List[Tensor], lse_tensors: List[Tensor],
                     use_autograd_fix: bool = True) -> Tuple[Tensor, Tensor]:
    """``use_autograd_fix`` is accepted for signature compatibility; the merge is
    built from differentiable tensor ops, so gradients are exact for any count."""
    if len(outputs) < 2:
        raise ValueError("merge_attentions expects at least two outputs.")
    if len(outputs) != len(lse_tensors):
        raise ValueError("Number of outputs and LSE tensors must match.")
    shape = outputs[0].shape
    for i, (o, l) in enumerate(zip(outputs, lse_tensors)):
        if o.shape != shape:
            raise ValueError(f"Output {i} shape {tuple(o.shape)} does not match output 0 shape {tuple(shape)}.")
        if l.shape != shape[:-1]:
            raise ValueError(f"LSE {i} shape {tuple(l.shape)} does not match expected {tuple(shape[:-1])}.")
    acc = torch.float64 if outputs[0].dtype == torch.float64 else torch.float32
    lse_all = torch.stack([l.to(acc) for l in lse_tensors], dim=0)
    merged_lse = torch.logsumexp(lse_all, dim=0)
    weights = torch.exp(lse_all - merged_lse.unsqueeze(0)).unsqueeze(-1)
    merged = (weights * torch.stack([o.to(acc) for o in outputs], dim=0)).sum(dim=0)
    return merged.to(outputs[0].dtype), merged_lse


__all__ = ["merge_attentions"]
