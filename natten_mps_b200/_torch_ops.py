"""``torch.library`` custom ops of the CUDA path, with autograd.

Namespace ``natten_b200``.  The rank-specific ops keep the schemas of the
reference's ``natten_mps::*`` ops (``src/natten_mps/_torch_ops.py:39-42, 82-85,
286-289, 583-586``) so code written against them only changes the namespace:

    na{1,2,3}d_qk(query, key, kernel_size, dilation, stride, is_causal, scale?) -> Tensor
    na{1,2,3}d_av(attn, value, kernel_size, dilation, stride, is_causal) -> Tensor
    na{1,2,3}d_fwd(query, key, value, kernel_size, stride, dilation, is_causal, scale?) -> Tensor
    na{1,2,3}d_varlen_fwd(query, key, value, sizes, kernel_size, dilation, scale?) -> Tensor

They are thin compositions of four rank-generic ops that own the kernels:

    na_fused      -> (out, lse)   fused forward; GQA, additional tokens, extents
    na_fused_bwd  -> (dq, dk, dv, d_extra_k, d_extra_v)
    na_qk / na_qk_bwd,  na_av / na_av_bwd

Only a ``CUDA`` implementation (plus ``Meta`` shape functions) is registered:
calling an op with CPU tensors fails in the dispatcher instead of silently
running something else.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import _backend

LIB = torch.library.Library("natten_b200", "DEF")
NS = "natten_b200"


def _strided(spatial: Sequence[int], stride: Sequence[int]) -> List[int]:
    return [(n - 1) // s + 1 for n, s in zip(spatial, stride)]


def _opt(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None or t.numel() == 0 else t


# ---------------------------------------------------------------------------
# rank-generic fused op
# ---------------------------------------------------------------------------
LIB.define(
    "na_fused(Tensor query, Tensor key, Tensor value, Tensor? extra_k, Tensor? extra_v, "
    "Tensor? extents, int[] kernel_size, int[] stride, int[] dilation, bool[] is_causal, "
    "float scale) -> (Tensor, Tensor)")
LIB.define(
    "na_fused_bwd(Tensor query, Tensor key, Tensor value, Tensor? extra_k, Tensor? extra_v, "
    "Tensor? extents, Tensor out, Tensor lse, Tensor dout, Tensor? dlse, int[] kernel_size, "
    "int[] stride, int[] dilation, bool[] is_causal, float scale) "
    "-> (Tensor, Tensor, Tensor, Tensor, Tensor)")


@torch.library.impl(LIB, "na_fused", "CUDA")
def _na_fused_cuda(query, key, value, extra_k, extra_v, extents, kernel_size, stride, dilation,
                   is_causal, scale):
    return _backend.fused_forward(query, key, value, tuple(kernel_size), tuple(stride),
                                  tuple(dilation), tuple(is_causal), float(scale),
                                  extra_k, extra_v, extents)


@torch.library.impl(LIB, "na_fused", "Meta")
def _na_fused_meta(query, key, value, extra_k, extra_v, extents, kernel_size, stride, dilation,
                   is_causal, scale):
    rank = query.ndim - 3
    osp = _strided(query.shape[1:1 + rank], stride)
    out = query.new_empty((query.shape[0], *osp, query.shape[-2], value.shape[-1]))
    acc = torch.float64 if query.dtype == torch.float64 else torch.float32
    lse = query.new_empty((query.shape[0], *osp, query.shape[-2]), dtype=acc)
    return out, lse


@torch.library.impl(LIB, "na_fused_bwd", "CUDA")
def _na_fused_bwd_cuda(query, key, value, extra_k, extra_v, extents, out, lse, dout, dlse,
                       kernel_size, stride, dilation, is_causal, scale):
    dq, dk, dv, dek, dev = _backend.fused_backward(
        query, key, value, out, lse, dout, tuple(kernel_size), tuple(stride), tuple(dilation),
        tuple(is_causal), float(scale), extra_k, extra_v, extents, dlse)
    if dek is None:
        dek = query.new_empty(0)
        dev = query.new_empty(0)
    return dq, dk, dv, dek, dev


@torch.library.impl(LIB, "na_fused_bwd", "Meta")
def _na_fused_bwd_meta(query, key, value, extra_k, extra_v, extents, out, lse, dout, dlse,
                       kernel_size, stride, dilation, is_causal, scale):
    dek = torch.empty_like(extra_k) if extra_k is not None else query.new_empty(0)
    dev = torch.empty_like(extra_v) if extra_v is not None else query.new_empty(0)
    return (query.new_empty(query.shape), key.new_empty(key.shape), value.new_empty(value.shape),
            dek, dev)


def _fused_setup(ctx, inputs, output):
    (q, k, v, ek, ev, extents, kernel_size, stride, dilation, is_causal, scale) = inputs
    out, lse = output
    ctx.geometry = (list(kernel_size), list(stride), list(dilation), list(is_causal), float(scale))
    ctx.has_extra = ek is not None
    ctx.has_extents = extents is not None
    saved = [q, k, v, out, lse]
    if ek is not None:
        saved += [ek, ev]
    if extents is not None:
        saved.append(extents)
    ctx.save_for_backward(*saved)


def _fused_backward(ctx, grad_out, grad_lse):
    saved = list(ctx.saved_tensors)
    q, k, v, out, lse = saved[:5]
    rest = saved[5:]
    ek = ev = extents = None
    if ctx.has_extra:
        ek, ev = rest[0], rest[1]
        rest = rest[2:]
    if ctx.has_extents:
        extents = rest[0]
    ks, st, dil, causal, scale = ctx.geometry
    if grad_out is None:
        grad_out = torch.zeros_like(out)
    dq, dk, dv, dek, dev = torch.ops.natten_b200.na_fused_bwd(
        q, k, v, ek, ev, extents, out, lse, grad_out, grad_lse, ks, st, dil, causal, scale)
    return (dq, dk, dv, dek if ctx.has_extra else None, dev if ctx.has_extra else None, None,
            None, None, None, None, None)


torch.library.register_autograd(f"{NS}::na_fused", _fused_backward, setup_context=_fused_setup)


# ---------------------------------------------------------------------------
# rank-generic split ops
# ---------------------------------------------------------------------------
LIB.define("na_qk(Tensor query, Tensor key, int[] kernel_size, int[] dilation, int[] stride, "
           "bool[] is_causal, float? scale) -> Tensor")
LIB.define("na_qk_bwd(Tensor dlogits, Tensor query, Tensor key, int[] kernel_size, int[] dilation, "
           "int[] stride, bool[] is_causal, float? scale) -> (Tensor, Tensor)")
LIB.define("na_av(Tensor attn, Tensor value, int[] kernel_size, int[] dilation, int[] stride, "
           "bool[] is_causal) -> Tensor")
LIB.define("na_av_bwd(Tensor dout, Tensor attn, Tensor value, int[] kernel_size, int[] dilation, "
           "int[] stride, bool[] is_causal) -> (Tensor, Tensor)")


@torch.library.impl(LIB, "na_qk", "CUDA")
def _na_qk_cuda(query, key, kernel_size, dilation, stride, is_causal, scale):
    return _backend.qk_forward(query, key, tuple(kernel_size), tuple(dilation), tuple(stride),
                               tuple(is_causal), scale)


@torch.library.impl(LIB, "na_qk", "Meta")
def _na_qk_meta(query, key, kernel_size, dilation, stride, is_causal, scale):
    rank = query.ndim - 3
    ktot = 1
    for x in kernel_size:
        ktot *= x
    return query.new_empty((query.shape[0], *_strided(query.shape[1:1 + rank], stride),
                            query.shape[-2], ktot))


@torch.library.impl(LIB, "na_qk_bwd", "CUDA")
def _na_qk_bwd_cuda(dlogits, query, key, kernel_size, dilation, stride, is_causal, scale):
    return _backend.qk_backward(dlogits, query, key, tuple(kernel_size), tuple(dilation),
                                tuple(stride), tuple(is_causal), scale)


@torch.library.impl(LIB, "na_qk_bwd", "Meta")
def _na_qk_bwd_meta(dlogits, query, key, kernel_size, dilation, stride, is_causal, scale):
    return query.new_empty(query.shape), key.new_empty(key.shape)


def _qk_setup(ctx, inputs, output):
    q, k, kernel_size, dilation, stride, is_causal, scale = inputs
    ctx.geometry = (list(kernel_size), list(dilation), list(stride), list(is_causal), scale)
    ctx.save_for_backward(q, k)


def _qk_backward(ctx, grad_logits):
    q, k = ctx.saved_tensors
    ks, dil, st, causal, scale = ctx.geometry
    dq, dk = torch.ops.natten_b200.na_qk_bwd(grad_logits, q, k, ks, dil, st, causal, scale)
    return dq, dk, None, None, None, None, None


torch.library.register_autograd(f"{NS}::na_qk", _qk_backward, setup_context=_qk_setup)


@torch.library.impl(LIB, "na_av", "CUDA")
def _na_av_cuda(attn, value, kernel_size, dilation, stride, is_causal):
    return _backend.av_forward(attn, value, tuple(kernel_size), tuple(dilation), tuple(stride),
                               tuple(is_causal))


@torch.library.impl(LIB, "na_av", "Meta")
def _na_av_meta(attn, value, kernel_size, dilation, stride, is_causal):
    return value.new_empty((*attn.shape[:-1], value.shape[-1]))


@torch.library.impl(LIB, "na_av_bwd", "CUDA")
def _na_av_bwd_cuda(dout, attn, value, kernel_size, dilation, stride, is_causal):
    return _backend.av_backward(dout, attn, value, tuple(kernel_size), tuple(dilation),
                                tuple(stride), tuple(is_causal))


@torch.library.impl(LIB, "na_av_bwd", "Meta")
def _na_av_bwd_meta(dout, attn, value, kernel_size, dilation, stride, is_causal):
    return attn.new_empty(attn.shape, dtype=value.dtype), value.new_empty(value.shape)


def _av_setup(ctx, inputs, output):
    attn, v, kernel_size, dilation, stride, is_causal = inputs
    ctx.geometry = (list(kernel_size), list(dilation), list(stride), list(is_causal))
    ctx.attn_dtype = attn.dtype
    ctx.save_for_backward(attn, v)


def _av_backward(ctx, grad_out):
    attn, v = ctx.saved_tensors
    ks, dil, st, causal = ctx.geometry
    dattn, dv = torch.ops.natten_b200.na_av_bwd(grad_out, attn, v, ks, dil, st, causal)
    return dattn.to(ctx.attn_dtype), dv, None, None, None, None


torch.library.register_autograd(f"{NS}::na_av", _av_backward, setup_context=_av_setup)


# ---------------------------------------------------------------------------
# rank-specific names with the reference's schemas
# ---------------------------------------------------------------------------
def _define_rank_ops(rank: int) -> None:
    LIB.define(f"na{rank}d_qk(Tensor query, Tensor key, int[] kernel_size, int[] dilation, "
               "int[] stride, bool[] is_causal, float? scale) -> Tensor")
    LIB.define(f"na{rank}d_av(Tensor attn, Tensor value, int[] kernel_size, int[] dilation, "
               "int[] stride, bool[] is_causal) -> Tensor")
    LIB.define(f"na{rank}d_fwd(Tensor query, Tensor key, Tensor value, int[] kernel_size, "
               "int[] stride, int[] dilation, bool[] is_causal, float? scale) -> Tensor")
    LIB.define(f"na{rank}d_varlen_fwd(Tensor query, Tensor key, Tensor value, Tensor sizes, "
               "int[] kernel_size, int[] dilation, float? scale) -> Tensor")

    def _check(t, what):
        if t.ndim != rank + 3:
            raise ValueError(f"na{rank}d {what} must have {rank + 3} dimensions, got {t.ndim}.")

    def qk(query, key, kernel_size, dilation, stride, is_causal, scale):
        _check(query, "query")
        return torch.ops.natten_b200.na_qk(query, key, kernel_size, dilation, stride, is_causal, scale)

    def av(attn, value, kernel_size, dilation, stride, is_causal):
        _check(value, "value")
        return torch.ops.natten_b200.na_av(attn, value, kernel_size, dilation, stride, is_causal)

    def fwd(query, key, value, kernel_size, stride, dilation, is_causal, scale):
        _check(query, "query")
        sc = float(query.shape[-1] ** -0.5 if scale is None else scale)
        return torch.ops.natten_b200.na_fused(query, key, value, None, None, None, kernel_size,
                                              stride, dilation, is_causal, sc)[0]

    def varlen_fwd(query, key, value, sizes, kernel_size, dilation, scale):
        _check(query, "query")
        sc = float(query.shape[-1] ** -0.5 if scale is None else scale)
        ones, no = [1] * rank, [False] * rank
        return torch.ops.natten_b200.na_fused(query, key, value, None, None, sizes, kernel_size,
                                              ones, dilation, no, sc)[0]

    for name, fn in ((f"na{rank}d_qk", qk), (f"na{rank}d_av", av), (f"na{rank}d_fwd", fwd),
                     (f"na{rank}d_varlen_fwd", varlen_fwd)):
        LIB.impl(name, fn, "CompositeImplicitAutograd")


for _rank in (1, 2, 3):
    _define_rank_ops(_rank)

OP_NAMES = ("na_fused", "na_fused_bwd", "na_qk", "na_qk_bwd", "na_av", "na_av_bwd") + tuple(
    f"na{r}d_{s}" for r in (1, 2, 3) for s in ("qk", "av", "fwd", "varlen_fwd"))
