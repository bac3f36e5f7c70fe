"""Parameter normalisation and the shape rules every entry point enforces.

Same accepted inputs, same ``ValueError`` conditions as the reference's
``src/natten_mps/utils/params.py:19-82`` (ints or per-axis sequences; values
positive; ``kernel <= extent``, ``stride <= kernel``, ``kernel * dilation <=
extent`` per axis).
"""
from __future__ import annotations

from collections.abc import Sequence


def normalize_tuple_param(param, rank: int, name: str):
    """int / bool / sequence -> tuple of length ``rank`` (all-bool or all positive int)."""
    if isinstance(param, (bool, int)):
        items = [param] * rank
    elif isinstance(param, Sequence) and not isinstance(param, (str, bytes)):
        items = list(param)
        if len(items) != rank:
            raise ValueError(f"{name} must have length {rank}, got {len(items)}.")
    else:
        raise ValueError(f"{name} must be an int, bool, or tuple/list of length {rank}.")

    flags = [isinstance(x, bool) for x in items]
    if all(flags):
        return tuple(bool(x) for x in items)
    if any(flags):
        raise ValueError(f"{name} cannot mix bool and int values.")
    for x in items:
        if not isinstance(x, int):
            raise ValueError(f"{name} values must be int or bool.")
        if x <= 0:
            raise ValueError(f"{name} values must be > 0, got {x}.")
    return tuple(int(x) for x in items)


def normalize_kernel_size(kernel_size, rank: int):
    values = normalize_tuple_param(kernel_size, rank, "kernel_size")
    if any(isinstance(x, bool) for x in values):
        raise ValueError("kernel_size must contain integers, not bools.")
    return values


def _same_rank(label_a, a, label_b, b):
    if len(a) != len(b):
        raise ValueError(f"{label_a} rank ({len(a)}) must match {label_b} rank ({len(b)}).")


def check_kernel_size_vs_input(kernel_size, input_spatial_shape):
    _same_rank("kernel_size", kernel_size, "input", input_spatial_shape)
    for axis, (k, n) in enumerate(zip(kernel_size, input_spatial_shape)):
        if k > n:
            raise ValueError(f"kernel_size[{axis}]={k} cannot exceed input spatial size {n}.")


def check_stride_vs_kernel(stride, kernel_size):
    _same_rank("stride", stride, "kernel_size", kernel_size)
    for axis, (s, k) in enumerate(zip(stride, kernel_size)):
        if s > k:
            raise ValueError(f"stride[{axis}]={s} must be <= kernel_size[{axis}]={k}.")


def check_dilation_kernel_vs_input(dilation, kernel_size, input_spatial_shape):
    if not (len(dilation) == len(kernel_size) == len(input_spatial_shape)):
        raise ValueError("dilation, kernel_size, and input_spatial_shape must share the same rank.")
    for axis, (d, k, n) in enumerate(zip(dilation, kernel_size, input_spatial_shape)):
        if d * k > n:
            raise ValueError(
                f"dilation[{axis}] * kernel_size[{axis}] = {d * k} exceeds input spatial size {n}.")
