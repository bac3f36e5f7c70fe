"""Functional API: ``na{1,2,3}d``, the split ``na{1,2,3}d_qk`` / ``na{1,2,3}d_av``
ops and ``na{1,2,3}d_varlen``.

Signatures, argument meaning, accepted shapes and ``ValueError`` conditions follow
the reference's ``src/natten_mps/functional.py`` (``na1d`` :213-303, ``na2d``
:306-394, ``na3d`` :522-611, split ops :397-519 / :614-675, varlen :898-1026).
What differs is underneath: one CUDA path.  GQA/MQA heads are mapped inside the
kernels (no ``repeat_interleave``), additional key/value tokens join the same
softmax inside the fused kernel (no second attention + merge), per-sample
extents are a kernel argument (no Python loop), and the backward is one fused
call.  The varlen entry points additionally accept GQA shapes and
``additional_keys`` / ``additional_values``.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch
import torch.nn.functional as F

from . import _torch_ops  # noqa: F401  (registers torch.ops.natten_b200.*)
from .utils.params import (
    check_dilation_kernel_vs_input,
    check_kernel_size_vs_input,
    check_stride_vs_kernel,
    normalize_kernel_size,
    normalize_tuple_param,
)

_LAYOUT = {1: "[B, L, H, D]", 2: "[B, H, W, heads, dim]", 3: "[B, D, H, W, heads, dim]"}
IntOrTuple = Union[int, Tuple[int, ...]]
BoolOrTuple = Union[bool, Tuple[bool, ...]]


def _causal_tuple(is_causal, rank: int) -> Tuple[bool, ...]:
    return tuple(bool(x) for x in normalize_tuple_param(is_causal, rank, "is_causal"))


def _check_qkv(query, key, value, rank: int) -> None:
    nd = rank + 3
    if query.ndim != nd or key.ndim != nd or value.ndim != nd:
        raise ValueError(f"na{rank}d expects query/key/value with shape {_LAYOUT[rank]}.")
    sq, sk, sv = query.shape[1:-2], key.shape[1:-2], value.shape[1:-2]
    if sq != sk or sq != sv:
        raise ValueError(f"Spatial dimensions must match: Q={tuple(sq)}, K={tuple(sk)}, V={tuple(sv)}.")
    if query.shape[0] != key.shape[0] or query.shape[0] != value.shape[0]:
        raise ValueError("Batch dimensions must match.")
    if query.shape[-1] != key.shape[-1]:
        raise ValueError(
            f"Head dim must match between Q and K: Q has {query.shape[-1]}, K has {key.shape[-1]}.")
    if key.shape[-2] != value.shape[-2]:
        raise ValueError(
            f"K and V must have same number of heads: K={key.shape[-2]}, V={value.shape[-2]}.")
    if query.shape[-2] % key.shape[-2] != 0:
        raise ValueError(
            f"heads_q ({query.shape[-2]}) must be divisible by heads_kv ({key.shape[-2]}) for GQA.")


def _check_additional(query, key, additional_keys, additional_values) -> bool:
    if additional_keys is None and additional_values is None:
        return False
    if additional_keys is None or additional_values is None:
        raise ValueError("additional_keys and additional_values must both be provided or both None.")
    if additional_keys.ndim != 4 or additional_values.ndim != 4:
        raise ValueError("additional_keys/additional_values must be 4D: [B, N_extra, heads_kv, dim].")
    if additional_keys.shape[0] != query.shape[0]:
        raise ValueError("additional_keys batch must match query batch.")
    if additional_values.shape[0] != query.shape[0]:
        raise ValueError("additional_values batch must match query batch.")
    if additional_keys.shape[-1] != query.shape[-1]:
        raise ValueError("additional_keys head dim must match query head dim.")
    if additional_values.shape[-1] != query.shape[-1]:
        raise ValueError("additional_values head dim must match query head dim.")
    if additional_keys.shape[-2] != additional_values.shape[-2]:
        raise ValueError("additional_keys and additional_values must have same number of heads.")
    if additional_keys.shape[1] != additional_values.shape[1]:
        raise ValueError("additional_keys and additional_values must have same N_extra.")
    if additional_keys.shape[-2] != key.shape[-2]:
        raise ValueError("additional_keys must have the same number of heads as key.")
    return True


def _global_attention(query, key, value, scale, return_lse, extra_k, extra_v):
    """Kernel covers the whole input on every axis: neighbourhood attention is plain
    global attention, which the reference hands to PyTorch's SDPA
    (src/natten_mps/functional.py:148-206).  Same here; it is not a neighbourhood
    computation, so no kernel of this library is involved."""
    B, Hq, D = query.shape[0], query.shape[-2], query.shape[-1]
    spatial = tuple(query.shape[1:-2])
    group = Hq // key.shape[-2]
    k_all = key.reshape(B, -1, key.shape[-2], D)
    v_all = value.reshape(B, -1, value.shape[-2], value.shape[-1])
    if extra_k is not None:
        k_all = torch.cat([k_all, extra_k], dim=1)
        v_all = torch.cat([v_all, extra_v], dim=1)
    q_t = query.reshape(B, -1, Hq, D).transpose(1, 2)
    k_t = k_all.transpose(1, 2).repeat_interleave(group, dim=1) if group > 1 else k_all.transpose(1, 2)
    v_t = v_all.transpose(1, 2).repeat_interleave(group, dim=1) if group > 1 else v_all.transpose(1, 2)
    out = F.scaled_dot_product_attention(q_t, k_t, v_t, scale=scale)
    out = out.transpose(1, 2).reshape(B, *spatial, Hq, value.shape[-1])
    if not return_lse:
        return out
    lse = torch.logsumexp(torch.matmul(q_t, k_t.transpose(-2, -1)) * scale, dim=-1)
    return out, lse.transpose(1, 2).reshape(B, *spatial, Hq)


def _na(rank, query, key, value, kernel_size, stride, dilation, is_causal, scale, return_lse,
        additional_keys, additional_values):
    _check_qkv(query, key, value, rank)
    has_extra = _check_additional(query, key, additional_keys, additional_values)
    ks = normalize_kernel_size(kernel_size, rank)
    st = normalize_tuple_param(stride, rank, "stride")
    dil = normalize_tuple_param(dilation, rank, "dilation")
    causal = _causal_tuple(is_causal, rank)
    spatial = tuple(query.shape[1:1 + rank])
    check_kernel_size_vs_input(ks, spatial)
    check_stride_vs_kernel(st, ks)
    check_dilation_kernel_vs_input(dil, ks, spatial)
    sc = query.shape[-1] ** -0.5 if scale is None else float(scale)

    if all(k >= n for k, n in zip(ks, spatial)) and all(s == 1 for s in st) and not any(causal):
        return _global_attention(query, key, value, sc, return_lse,
                                 additional_keys if has_extra else None,
                                 additional_values if has_extra else None)

    out, lse = torch.ops.natten_b200.na_fused(
        query, key, value, additional_keys if has_extra else None,
        additional_values if has_extra else None, None, list(ks), list(st), list(dil),
        list(causal), sc)
    if not return_lse:
        return out
    # the reference returns the lse in the input dtype, and in float32 once the
    # additional tokens were merged in (src/natten_mps/merge.py:63-75)
    return out, (lse if has_extra else lse.to(query.dtype))


def na1d(query, key, value, kernel_size: IntOrTuple, stride: IntOrTuple = 1,
         dilation: IntOrTuple = 1, is_causal: BoolOrTuple = False, scale: Optional[float] = None,
         return_lse: bool = False, additional_keys: Optional[torch.Tensor] = None,
         additional_values: Optional[torch.Tensor] = None):
    """1-D neighbourhood attention.  ``query [B, L, Hq, D]``, ``key/value [B, L, Hkv, D]``
    with ``Hq % Hkv == 0``; returns ``[B, ceil(L/stride), Hq, D]`` (and the
    log-sum-exp ``[B, L_out, Hq]`` when ``return_lse``)."""
    return _na(1, query, key, value, kernel_size, stride, dilation, is_causal, scale, return_lse,
               additional_keys, additional_values)


def na2d(query, key, value, kernel_size: IntOrTuple, stride: IntOrTuple = 1,
         dilation: IntOrTuple = 1, is_causal: BoolOrTuple = False, scale: Optional[float] = None,
         return_lse: bool = False, additional_keys: Optional[torch.Tensor] = None,
         additional_values: Optional[torch.Tensor] = None):
    """2-D neighbourhood attention on ``[B, H, W, heads, dim]`` tensors."""
    return _na(2, query, key, value, kernel_size, stride, dilation, is_causal, scale, return_lse,
               additional_keys, additional_values)


def na3d(query, key, value, kernel_size: IntOrTuple, stride: IntOrTuple = 1,
         dilation: IntOrTuple = 1, is_causal: BoolOrTuple = False, scale: Optional[float] = None,
         return_lse: bool = False, additional_keys: Optional[torch.Tensor] = None,
         additional_values: Optional[torch.Tensor] = None):
    """3-D neighbourhood attention on ``[B, D, H, W, heads, dim]`` tensors."""
    return _na(3, query, key, value, kernel_size, stride, dilation, is_causal, scale, return_lse,
               additional_keys, additional_values)


# ---------------------------------------------------------------------------
# split ops
# ---------------------------------------------------------------------------
def _na_qk(rank, query, key, kernel_size, dilation, stride, is_causal, scale):
    if query.ndim != rank + 3 or key.ndim != rank + 3:
        raise ValueError(f"na{rank}d_qk expects query/key with shape {_LAYOUT[rank]}.")
    if query.shape != key.shape:
        raise ValueError(f"query and key must share the same shape in na{rank}d_qk.")
    ks = normalize_kernel_size(kernel_size, rank)
    dil = normalize_tuple_param(dilation, rank, "dilation")
    st = normalize_tuple_param(stride, rank, "stride")
    causal = _causal_tuple(is_causal, rank)
    spatial = tuple(query.shape[1:1 + rank])
    check_kernel_size_vs_input(ks, spatial)
    check_dilation_kernel_vs_input(dil, ks, spatial)
    return torch.ops.natten_b200.na_qk(query, key, list(ks), list(dil), list(st), list(causal),
                                       None if scale is None else float(scale))


def _na_av(rank, attn, value, kernel_size, dilation, stride, is_causal):
    names = {1: "[B, L, H, K]", 2: "[B, H, W, heads, K]", 3: "[B, D, H, W, heads, K]"}
    if attn.ndim != rank + 3:
        raise ValueError(f"na{rank}d_av expects attn with shape {names[rank]}.")
    if value.ndim != rank + 3:
        raise ValueError(f"na{rank}d_av expects value with shape {_LAYOUT[rank]}.")
    if attn.shape[0] != value.shape[0] or attn.shape[-2] != value.shape[-2]:
        raise ValueError(f"na{rank}d_av requires attn/value to match on batch and heads dimensions.")
    if any(a > n for a, n in zip(attn.shape[1:1 + rank], value.shape[1:1 + rank])):
        raise ValueError(f"na{rank}d_av attn spatial size cannot exceed value spatial size.")
    ks = normalize_kernel_size(kernel_size, rank)
    dil = normalize_tuple_param(dilation, rank, "dilation")
    st = normalize_tuple_param(stride, rank, "stride")
    causal = _causal_tuple(is_causal, rank)
    ktot = 1
    for x in ks:
        ktot *= x
    if attn.shape[-1] != ktot:
        what = {1: "kernel_size", 2: "kernel area", 3: "kernel volume"}[rank]
        raise ValueError(f"na{rank}d_av attn last dim ({attn.shape[-1]}) must match {what} ({ktot}).")
    spatial = tuple(value.shape[1:1 + rank])
    check_kernel_size_vs_input(ks, spatial)
    check_dilation_kernel_vs_input(dil, ks, spatial)
    expect = tuple((n + s - 1) // s for n, s in zip(spatial, st))
    if tuple(attn.shape[1:1 + rank]) != expect:
        raise ValueError(
            f"na{rank}d_av attn spatial size {tuple(attn.shape[1:1 + rank])} does not match "
            f"ceil(value spatial / stride) = {expect}.")
    return torch.ops.natten_b200.na_av(attn, value, list(ks), list(dil), list(st), list(causal))


def na1d_qk(query, key, kernel_size: IntOrTuple, dilation: IntOrTuple = 1, *,
            stride: IntOrTuple = 1, is_causal: BoolOrTuple = False, scale: Optional[float] = None):
    """Neighbourhood logits ``[B, L_out, H, K]``: unscaled dot products unless ``scale``
    is given; masked (causal) slots hold ``-inf``."""
    return _na_qk(1, query, key, kernel_size, dilation, stride, is_causal, scale)


def na2d_qk(query, key, kernel_size: IntOrTuple, dilation: IntOrTuple = 1, *,
            stride: IntOrTuple = 1, is_causal: BoolOrTuple = False, scale: Optional[float] = None):
    return _na_qk(2, query, key, kernel_size, dilation, stride, is_causal, scale)


def na3d_qk(query, key, kernel_size: IntOrTuple, dilation: IntOrTuple = 1, *,
            stride: IntOrTuple = 1, is_causal: BoolOrTuple = False, scale: Optional[float] = None):
    return _na_qk(3, query, key, kernel_size, dilation, stride, is_causal, scale)


class _QKRPB(torch.autograd.Function):
    """Split QK with a relative position bias (``src/natten_mps/compat/v014.py:66-183``)."""

    @staticmethod
    def forward(ctx, query, key, rpb, ks, dil, scale):
        from . import _backend
        ctx.save_for_backward(query, key)
        ctx.geo = (ks, dil, scale, tuple(rpb.shape), rpb.dtype)
        return _backend.qk_rpb_forward(query, key, rpb, ks, dil, scale)

    @staticmethod
    def backward(ctx, grad_logits):
        from . import _backend
        query, key = ctx.saved_tensors
        ks, dil, scale, rpb_shape, rpb_dtype = ctx.geo
        dq, dk, drpb = _backend.qk_rpb_backward(grad_logits, query, key, rpb_shape, ks, dil, scale)
        return dq, dk, drpb.to(rpb_dtype), None, None, None


def _na_qk_rpb(rank, query, key, rpb, kernel_size, dilation, scale):
    if query.ndim != rank + 3 or key.ndim != rank + 3:
        raise ValueError(f"na{rank}d_qk_rpb expects query/key with shape {_LAYOUT[rank]}.")
    if query.shape != key.shape:
        raise ValueError("query and key must have identical shapes.")
    ks = normalize_kernel_size(kernel_size, rank)
    dil = normalize_tuple_param(dilation, rank, "dilation")
    spatial = tuple(query.shape[1:1 + rank])
    check_kernel_size_vs_input(ks, spatial)
    check_dilation_kernel_vs_input(dil, ks, spatial)
    if any(x % 2 == 0 for x in ks):
        # with an even kernel the bias window start reaches K, so start + slot runs one past the 2K-1 entries
        # (the reference's table lookup fails there as well)
        raise ValueError("relative position bias needs odd kernel sizes.")
    want = (query.shape[-2], *[2 * x - 1 for x in ks])
    if tuple(rpb.shape) != want:
        raise ValueError(f"rpb must have shape {list(want)} for {rank}D.")
    return _QKRPB.apply(query, key, rpb, ks, dil, None if scale is None else float(scale))


def na1d_qk_rpb(query, key, rpb, kernel_size: IntOrTuple, dilation: IntOrTuple = 1, *,
                scale: Optional[float] = None):
    """``na1d_qk`` plus a relative position bias ``rpb [H, 2K-1]``: slot ``j`` of position ``i`` adds
    ``rpb[h, get_pb_start(i) + j]`` (heads-last form of the reference's ``natten1dqkrpb``)."""
    return _na_qk_rpb(1, query, key, rpb, kernel_size, dilation, scale)


def na2d_qk_rpb(query, key, rpb, kernel_size: IntOrTuple, dilation: IntOrTuple = 1, *,
                scale: Optional[float] = None):
    """``na2d_qk`` plus ``rpb [H, 2Kh-1, 2Kw-1]`` (heads-last form of ``natten2dqkrpb``)."""
    return _na_qk_rpb(2, query, key, rpb, kernel_size, dilation, scale)


def na3d_qk_rpb(query, key, rpb, kernel_size: IntOrTuple, dilation: IntOrTuple = 1, *,
                scale: Optional[float] = None):
    """``na3d_qk`` plus ``rpb [H, 2Kd-1, 2Kh-1, 2Kw-1]``."""
    return _na_qk_rpb(3, query, key, rpb, kernel_size, dilation, scale)


def na1d_av(attn, value, kernel_size: IntOrTuple, dilation: IntOrTuple = 1, *,
            stride: IntOrTuple = 1, is_causal: BoolOrTuple = False):
    """Weighted sum of neighbourhood values: ``attn [B, L_out, H, K]``, ``value [B, L, H, Dv]``."""
    return _na_av(1, attn, value, kernel_size, dilation, stride, is_causal)


def na2d_av(attn, value, kernel_size: IntOrTuple, dilation: IntOrTuple = 1, *,
            stride: IntOrTuple = 1, is_causal: BoolOrTuple = False):
    return _na_av(2, attn, value, kernel_size, dilation, stride, is_causal)


def na3d_av(attn, value, kernel_size: IntOrTuple, dilation: IntOrTuple = 1, *,
            stride: IntOrTuple = 1, is_causal: BoolOrTuple = False):
    return _na_av(3, attn, value, kernel_size, dilation, stride, is_causal)


# ---------------------------------------------------------------------------
# variable-length
# ---------------------------------------------------------------------------
def _check_sizes(sizes: torch.Tensor, batch: int, max_spatial, ks, rank: int) -> torch.Tensor:
    if rank == 1:
        if sizes.ndim != 1 or sizes.shape[0] != batch:
            raise ValueError(
                f"seq_lens must be a 1-D tensor of length B={batch}, got shape {tuple(sizes.shape)}.")
        label = "seq_lens"
    else:
        if sizes.ndim != 2 or sizes.shape[0] != batch or sizes.shape[1] != rank:
            raise ValueError(
                f"spatial_sizes must be a [B, {rank}] tensor, got shape {tuple(sizes.shape)}.")
        label = "spatial_sizes"
    if sizes.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"{label} must be int32 or int64, got {sizes.dtype}.")
    table = sizes.reshape(batch, rank)
    if batch > 0:
        lo = table.amin(dim=0).tolist()      # one host read, like the reference's .item() checks
        hi = table.amax(dim=0).tolist()
        for a in range(rank):
            if rank == 1:
                if lo[a] < ks[a]:
                    raise ValueError(
                        f"All seq_lens must be >= kernel_size ({ks[a]}), but min(seq_lens)={lo[a]}.")
                if hi[a] > max_spatial[a]:
                    raise ValueError(
                        f"All seq_lens must be <= L_max ({max_spatial[a]}), but max(seq_lens)={hi[a]}.")
            else:
                if lo[a] < ks[a]:
                    raise ValueError(
                        f"All spatial_sizes[:,{a}] must be >= kernel_size[{a}] ({ks[a]}), but min={lo[a]}.")
                if hi[a] > max_spatial[a]:
                    raise ValueError(
                        f"All spatial_sizes[:,{a}] must be <= max_spatial[{a}] ({max_spatial[a]}), "
                        f"but max={hi[a]}.")
    return table.to(torch.int32)


def _na_varlen(rank, query, key, value, sizes, kernel_size, dilation, scale, additional_keys,
               additional_values):
    if query.ndim != rank + 3 or key.ndim != rank + 3 or value.ndim != rank + 3:
        raise ValueError(f"na{rank}d_varlen expects query/key/value with shape {_LAYOUT[rank]}.")
    if query.shape[:-2] != key.shape[:-2] or key.shape != value.shape or query.shape[-1] != key.shape[-1] \
            or query.shape[-2] % key.shape[-2] != 0:
        raise ValueError("query, key, and value must have identical shapes "
                         "(key/value may carry fewer heads when heads_q is divisible by heads_kv).")
    has_extra = _check_additional(query, key, additional_keys, additional_values)
    ks = normalize_kernel_size(kernel_size, rank)
    dil = normalize_tuple_param(dilation, rank, "dilation")
    spatial = tuple(query.shape[1:1 + rank])
    extents = _check_sizes(sizes, query.shape[0], spatial, ks, rank)
    sc = query.shape[-1] ** -0.5 if scale is None else float(scale)
    out, _ = torch.ops.natten_b200.na_fused(
        query, key, value, additional_keys if has_extra else None,
        additional_values if has_extra else None, extents, list(ks), [1] * rank, list(dil),
        [False] * rank, sc)
    return out


def na1d_varlen(query, key, value, seq_lens: torch.Tensor, kernel_size: IntOrTuple,
                dilation: IntOrTuple = 1, scale: Optional[float] = None, *,
                additional_keys: Optional[torch.Tensor] = None,
                additional_values: Optional[torch.Tensor] = None):
    """Padded batch ``[B, L_max, H, D]`` where sample ``b`` only has ``seq_lens[b]``
    tokens (``kernel_size <= seq_lens[b] <= L_max``).  Windows are computed against
    the sample's own length; rows past it are zero in the output and get zero grads."""
    return _na_varlen(1, query, key, value, seq_lens, kernel_size, dilation, scale,
                      additional_keys, additional_values)


def na2d_varlen(query, key, value, spatial_sizes: torch.Tensor, kernel_size: IntOrTuple,
                dilation: IntOrTuple = 1, scale: Optional[float] = None, *,
                additional_keys: Optional[torch.Tensor] = None,
                additional_values: Optional[torch.Tensor] = None):
    return _na_varlen(2, query, key, value, spatial_sizes, kernel_size, dilation, scale,
                      additional_keys, additional_values)


def na3d_varlen(query, key, value, spatial_sizes: torch.Tensor, kernel_size: IntOrTuple,
                dilation: IntOrTuple = 1, scale: Optional[float] = None, *,
                additional_keys: Optional[torch.Tensor] = None,
                additional_values: Optional[torch.Tensor] = None):
    return _na_varlen(3, query, key, value, spatial_sizes, kernel_size, dilation, scale,
                      additional_keys, additional_values)


__all__ = [
    "na1d_qk_rpb", "na2d_qk_rpb", "na3d_qk_rpb",
    "na1d", "na2d", "na3d", "na1d_qk", "na1d_av", "na2d_qk", "na2d_av", "na3d_qk", "na3d_av",
    "na1d_varlen", "na2d_varlen", "na3d_varlen",
]
