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


def get_pb_start(index: int, length: int, kernel_size: int, dilation: int) -> int:
    """First entry of the relative-position-bias window of ``index``: slot ``j`` of the position's
    neighbourhood reads bias entry ``get_pb_start(...) + j`` of a table with ``2 * kernel_size - 1``
    entries per axis (reference: ``src/natten_mps/utils/window.py:119-135``)."""
    half = kernel_size // 2
    if dilation <= 1:
        if index < half:
            return half + (half - index)
        if index + half >= length:
            return half + (length - index - 1 - half)
        return half
    if index - half * dilation < 0:
        return kernel_size - 1 - index // dilation
    if index + half * dilation >= length:
        return (length - index - 1) // dilation
    return half


def get_pb_start_vectorized(indices: torch.Tensor, length: int, kernel_size: int,
                            dilation: int) -> torch.Tensor:
    """Tensor form of :func:`get_pb_start` (reference: ``src/natten_mps/utils/window.py:49-83``)."""
    idx = indices.to(torch.long)
    half = kernel_size // 2
    mid = torch.full_like(idx, half)
    if dilation <= 1:
        left = torch.where(idx < half, half - idx, torch.zeros_like(idx))
        right = torch.where(idx + half >= length, length - idx - 1 - half, torch.zeros_like(idx))
        return mid + left + right
    out = torch.where(idx + half * dilation >= length, torch.div(length - idx - 1, dilation, rounding_mode="floor"), mid)
    return torch.where(idx - half * dilation < 0, kernel_size - 1 - torch.div(idx, dilation, rounding_mode="floor"), out)
