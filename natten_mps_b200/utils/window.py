"""Host-side copy of the window arithmetic the kernels implement.

``get_window_start`` is the integer specification of the neighbourhood
(reference: ``src/natten_mps/utils/window.py:91-111``); the CUDA kernels carry
the same function (``csrc/geometry.cuh``).  These helpers exist for users who
need the window positions on the host (visualisation, masks, tests).
"""
from __future__ import annotations

import torch


def get_window_start(index: int, length: int, kernel_size: int, dilation: int) -> int:
    half = kernel_size // 2
    if dilation <= 1:
        start = max(index - half, 0)
        if index + half >= length:
            start += length - index - half - 1
        return start
    reach = half * dilation
    if index - reach < 0:
        return index % dilation
    if index + reach >= length:
        phase = index % dilation
        full = (length // dilation) * dilation
        tail = length - full
        if phase < tail:
            return length - tail + phase - 2 * reach
        return full + phase - kernel_size * dilation
    return index - reach


def get_window_end(index: int, length: int, kernel_size: int, dilation: int) -> int:
    """Inclusive last position of the window."""
    return get_window_start(index, length, kernel_size, dilation) + (kernel_size - 1) * dilation


def get_window_start_vectorized(indices: torch.Tensor, length: int, kernel_size: int,
                                dilation: int) -> torch.Tensor:
    idx = indices.to(torch.long)
    half = kernel_size // 2
    if dilation <= 1:
        start = (idx - half).clamp_min(0)
        return torch.where(idx + half >= length, start + (length - idx - half - 1), start)
    reach = half * dilation
    phase = torch.remainder(idx, dilation)
    full = (length // dilation) * dilation
    tail = length - full
    right = torch.where(phase < tail, length - tail + phase - 2 * reach,
                        full + phase - kernel_size * dilation)
    out = torch.where(idx + reach >= length, right, idx - reach)
    return torch.where(idx - reach < 0, phase, out)
