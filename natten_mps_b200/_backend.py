"""Tensor-level front end of the C ABI: allocates outputs with PyTorch, fills the
params struct and launches on the current CUDA stream.

The functions here take already-validated, already-normalised arguments (tuples
per axis).  They accept GQA shapes, additional key/value tokens and per-sample
extents directly, so the callers never expand heads or loop over samples.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from . import _cabi


def _require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "natten_mps_b200 runs on CUDA tensors only (there is no CPU fallback); "
                f"got a tensor on {t.device}")


def _out_spatial(spatial: Sequence[int], stride: Sequence[int]) -> Tuple[int, ...]:
    return tuple((n + s - 1) // s for n, s in zip(spatial, stride))


def _acc_dtype(dtype: torch.dtype) -> torch.dtype:
    return torch.float64 if dtype == torch.float64 else torch.float32


def _extents_tensor(extents: Optional[torch.Tensor], rank: int, device) -> Optional[torch.Tensor]:
    if extents is None:
        return None
    e = extents.to(device=device, dtype=torch.int32).reshape(-1, rank).contiguous()
    return e


def fused_forward(q, k, v, kernel_size, stride, dilation, is_causal, scale: float,
                  extra_k=None, extra_v=None, extents=None):
    """-> (out [B,*O,Hq,Dv], lse [B,*O,Hq] float32/float64)."""
    _require_cuda(q, k, v, extra_k, extra_v)
    rank = q.ndim - 3
    spatial = tuple(q.shape[1:1 + rank])
    B, Hq, D = q.shape[0], q.shape[-2], q.shape[-1]
    Hkv, Dv = k.shape[-2], v.shape[-1]
    q, qs = _cabi.as_strided_input(q, rank)
    k, ks_ = _cabi.as_strided_input(k, rank)
    v, vs = _cabi.as_strided_input(v, rank)
    n_extra = 0
    if extra_k is not None:
        extra_k, extra_v = extra_k.contiguous(), extra_v.contiguous()
        n_extra = extra_k.shape[1]
    ext = _extents_tensor(extents, rank, q.device)
    osp = _out_spatial(spatial, stride)
    out = torch.empty((B, *osp, Hq, Dv), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, *osp, Hq), dtype=_acc_dtype(q.dtype), device=q.device)
    p = _cabi.make_params(rank, q.dtype, B, Hq, Hkv, D, Dv, spatial, kernel_size, stride, dilation,
                          is_causal, scale, n_extra, qs, ks_, vs, ext)
    _cabi.poll_status(q.device)
    with torch.cuda.device(q.device):
        rc = _cabi.lib().natten_fused_fwd(p, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v),
                                          _cabi.ptr(extra_k), _cabi.ptr(extra_v), _cabi.ptr(out),
                                          _cabi.ptr(lse), _cabi.stream_of(q))
    _cabi.check(rc, "natten_fused_fwd")
    _cabi.track_status(q)
    return out, lse


def fused_backward(q, k, v, out, lse, dout, kernel_size, stride, dilation, is_causal, scale: float,
                   extra_k=None, extra_v=None, extents=None, dlse=None):
    """-> (dq, dk, dv, d_extra_k, d_extra_v)."""
    _require_cuda(q, k, v, out, lse, dout, extra_k, extra_v, dlse)
    rank = q.ndim - 3
    spatial = tuple(q.shape[1:1 + rank])
    B, Hq, D = q.shape[0], q.shape[-2], q.shape[-1]
    Hkv, Dv = k.shape[-2], v.shape[-1]
    q, qs = _cabi.as_strided_input(q, rank)
    k, ks_ = _cabi.as_strided_input(k, rank)
    v, vs = _cabi.as_strided_input(v, rank)
    out, dout, lse = out.contiguous(), dout.contiguous(), lse.contiguous()
    if dout.dtype != q.dtype:
        dout = dout.to(q.dtype)
    if dlse is not None:
        dlse = dlse.to(lse.dtype).contiguous()
    n_extra = 0
    dek = dev = None
    if extra_k is not None:
        extra_k, extra_v = extra_k.contiguous(), extra_v.contiguous()
        n_extra = extra_k.shape[1]
        dek, dev = torch.empty_like(extra_k), torch.empty_like(extra_v)
    ext = _extents_tensor(extents, rank, q.device)
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    dk = torch.empty(k.shape, dtype=k.dtype, device=q.device)
    dv = torch.empty(v.shape, dtype=v.dtype, device=q.device)
    p = _cabi.make_params(rank, q.dtype, B, Hq, Hkv, D, Dv, spatial, kernel_size, stride, dilation,
                          is_causal, scale, n_extra, qs, ks_, vs, ext)
    L = _cabi.lib()
    ws_bytes = int(L.natten_workspace_bytes(p, _cabi.OP_FUSED_BWD))
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=q.device)
    _cabi.poll_status(q.device)
    with torch.cuda.device(q.device):
        rc = L.natten_fused_bwd(p, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(extra_k),
                                _cabi.ptr(extra_v), _cabi.ptr(out), _cabi.ptr(lse), _cabi.ptr(dout),
                                _cabi.ptr(dlse), _cabi.ptr(dq), _cabi.ptr(dk), _cabi.ptr(dv),
                                _cabi.ptr(dek), _cabi.ptr(dev), _cabi.ptr(ws), ws.numel(),
                                _cabi.stream_of(q))
    _cabi.check(rc, "natten_fused_bwd")
    _cabi.track_status(q)
    return dq, dk, dv, dek, dev


def qk_forward(q, k, kernel_size, dilation, stride, is_causal, scale: Optional[float]):
    _require_cuda(q, k)
    rank = q.ndim - 3
    spatial = tuple(q.shape[1:1 + rank])
    B, Hq, D = q.shape[0], q.shape[-2], q.shape[-1]
    q, qs = _cabi.as_strided_input(q, rank)
    k, ks_ = _cabi.as_strided_input(k, rank)
    ktot = 1
    for x in kernel_size:
        ktot *= x
    logits = torch.empty((B, *_out_spatial(spatial, stride), Hq, ktot), dtype=q.dtype, device=q.device)
    p = _cabi.make_params(rank, q.dtype, B, Hq, k.shape[-2], D, D, spatial, kernel_size, stride,
                          dilation, is_causal, scale, 0, qs, ks_, ks_)
    _cabi.poll_status(q.device)
    with torch.cuda.device(q.device):
        rc = _cabi.lib().natten_qk_fwd(p, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(logits),
                                       _cabi.stream_of(q))
    _cabi.check(rc, "natten_qk_fwd")
    _cabi.track_status(q)
    return logits


def qk_backward(dlogits, q, k, kernel_size, dilation, stride, is_causal, scale: Optional[float]):
    _require_cuda(dlogits, q, k)
    rank = q.ndim - 3
    spatial = tuple(q.shape[1:1 + rank])
    B, Hq, D = q.shape[0], q.shape[-2], q.shape[-1]
    q, qs = _cabi.as_strided_input(q, rank)
    k, ks_ = _cabi.as_strided_input(k, rank)
    dlogits = dlogits.to(q.dtype).contiguous()
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    dk = torch.empty(k.shape, dtype=k.dtype, device=q.device)
    p = _cabi.make_params(rank, q.dtype, B, Hq, k.shape[-2], D, D, spatial, kernel_size, stride,
                          dilation, is_causal, scale, 0, qs, ks_, ks_)
    _cabi.poll_status(q.device)
    with torch.cuda.device(q.device):
        rc = _cabi.lib().natten_qk_bwd(p, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(dlogits),
                                       _cabi.ptr(dq), _cabi.ptr(dk), _cabi.stream_of(q))
    _cabi.check(rc, "natten_qk_bwd")
    _cabi.track_status(q)
    return dq, dk


def _av_params(attn, v, kernel_size, dilation, stride, is_causal, vs):
    rank = v.ndim - 3
    spatial = tuple(v.shape[1:1 + rank])
    return _cabi.make_params(rank, v.dtype, v.shape[0], attn.shape[-2], v.shape[-2], v.shape[-1],
                             v.shape[-1], spatial, kernel_size, stride, dilation, is_causal, None,
                             0, vs, vs, vs)


def av_forward(attn, v, kernel_size, dilation, stride, is_causal):
    _require_cuda(attn, v)
    rank = v.ndim - 3
    v, vs = _cabi.as_strided_input(v, rank)
    attn = attn.to(v.dtype).contiguous()
    out = torch.empty((*attn.shape[:-1], v.shape[-1]), dtype=v.dtype, device=v.device)
    p = _av_params(attn, v, kernel_size, dilation, stride, is_causal, vs)
    _cabi.poll_status(v.device)
    with torch.cuda.device(v.device):
        rc = _cabi.lib().natten_av_fwd(p, _cabi.ptr(attn), _cabi.ptr(v), _cabi.ptr(out),
                                       _cabi.stream_of(v))
    _cabi.check(rc, "natten_av_fwd")
    _cabi.track_status(v)
    return out


def av_backward(dout, attn, v, kernel_size, dilation, stride, is_causal):
    _require_cuda(dout, attn, v)
    rank = v.ndim - 3
    v, vs = _cabi.as_strided_input(v, rank)
    attn = attn.to(v.dtype).contiguous()
    dout = dout.to(v.dtype).contiguous()
    dattn = torch.empty_like(attn)
    dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    p = _av_params(attn, v, kernel_size, dilation, stride, is_causal, vs)
    _cabi.poll_status(v.device)
    with torch.cuda.device(v.device):
        rc = _cabi.lib().natten_av_bwd(p, _cabi.ptr(attn), _cabi.ptr(v), _cabi.ptr(dout),
                                       _cabi.ptr(dattn), _cabi.ptr(dv), _cabi.stream_of(v))
    _cabi.check(rc, "natten_av_bwd")
    _cabi.track_status(v)
    return dattn, dv


def qk_rpb_forward(q, k, rpb, kernel_size, dilation, scale: Optional[float]):
    """Logits with a relative position bias; ``rpb [H, 2*K_0-1, ...]``."""
    _require_cuda(q, k, rpb)
    rank = q.ndim - 3
    spatial = tuple(q.shape[1:1 + rank])
    B, Hq, D = q.shape[0], q.shape[-2], q.shape[-1]
    q, qs = _cabi.as_strided_input(q, rank)
    k, ks_ = _cabi.as_strided_input(k, rank)
    rpb = rpb.to(q.dtype).contiguous()
    ktot = 1
    for x in kernel_size:
        ktot *= x
    ones, no = (1,) * rank, (False,) * rank
    logits = torch.empty((B, *spatial, Hq, ktot), dtype=q.dtype, device=q.device)
    p = _cabi.make_params(rank, q.dtype, B, Hq, k.shape[-2], D, D, spatial, kernel_size, ones, dilation, no,
                          scale, 0, qs, ks_, ks_)
    _cabi.poll_status(q.device)
    with torch.cuda.device(q.device):
        rc = _cabi.lib().natten_qk_rpb_fwd(p, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(rpb), _cabi.ptr(logits),
                                           _cabi.stream_of(q))
    _cabi.check(rc, "natten_qk_rpb_fwd")
    _cabi.track_status(q)
    return logits


def qk_rpb_backward(dlogits, q, k, rpb_shape, kernel_size, dilation, scale: Optional[float]):
    """-> (dq, dk, d_rpb)."""
    _require_cuda(dlogits, q, k)
    rank = q.ndim - 3
    spatial = tuple(q.shape[1:1 + rank])
    B, Hq, D = q.shape[0], q.shape[-2], q.shape[-1]
    q, qs = _cabi.as_strided_input(q, rank)
    k, ks_ = _cabi.as_strided_input(k, rank)
    dlogits = dlogits.to(q.dtype).contiguous()
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    dk = torch.empty(k.shape, dtype=k.dtype, device=q.device)
    drpb = torch.empty(tuple(rpb_shape), dtype=q.dtype, device=q.device)
    ones, no = (1,) * rank, (False,) * rank
    p = _cabi.make_params(rank, q.dtype, B, Hq, k.shape[-2], D, D, spatial, kernel_size, ones, dilation, no,
                          scale, 0, qs, ks_, ks_)
    _cabi.poll_status(q.device)
    with torch.cuda.device(q.device):
        rc = _cabi.lib().natten_qk_rpb_bwd(p, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(dlogits), _cabi.ptr(dq),
                                           _cabi.ptr(dk), _cabi.ptr(drpb), _cabi.stream_of(q))
    _cabi.check(rc, "natten_qk_rpb_bwd")
    _cabi.track_status(q)
    return dq, dk, drpb
