"""The v0.14-era operators with relative position bias, heads-first layout.

Same signatures and layouts as ``src/natten_mps/compat/v014.py:66-183`` of the reference
(``natten1dqkrpb`` / ``natten1dav`` / ``natten2dqkrpb`` / ``natten2dav``); the tensors are permuted to
the heads-last layout the kernels use (a view for the inputs, one copy for the result) and the bias is
added by the library's relative-position-bias kernels.
"""
from __future__ import annotations

import torch

from .. import functional as F


def natten1dqkrpb(query, key, rpb, kernel_size, dilation):
    """query, key ``[B, H, L, D]``, rpb ``[H, 2K-1]`` -> logits ``[B, H, L, K]``."""
    if query.ndim != 4 or key.ndim != 4:
        raise ValueError("natten1dqkrpb expects query/key shape [B, H, L, D].")
    if query.shape != key.shape:
        raise ValueError("query and key must have identical shapes.")
    out = F.na1d_qk_rpb(query.permute(0, 2, 1, 3), key.permute(0, 2, 1, 3), rpb, kernel_size, dilation)
    return out.permute(0, 2, 1, 3)


def natten1dav(attn, value, kernel_size, dilation):
    """attn ``[B, H, L, K]``, value ``[B, H, L, D]`` -> ``[B, H, L, D]``."""
    if attn.ndim != 4 or value.ndim != 4:
        raise ValueError("natten1dav expects attn [B,H,L,K] and value [B,H,L,D].")
    out = F.na1d_av(attn.permute(0, 2, 1, 3), value.permute(0, 2, 1, 3), kernel_size, dilation)
    return out.permute(0, 2, 1, 3)


def natten2dqkrpb(query, key, rpb, kernel_size, dilation):
    """query, key ``[B, H, Hh, Hw, D]``, rpb ``[H, 2Kh-1, 2Kw-1]`` -> ``[B, H, Hh, Hw, Kh*Kw]``."""
    if query.ndim != 5 or key.ndim != 5:
        raise ValueError("natten2dqkrpb expects query/key shape [B, H, Hh, Hw, D].")
    if query.shape != key.shape:
        raise ValueError("query and key must have identical shapes.")
    out = F.na2d_qk_rpb(query.permute(0, 2, 3, 1, 4), key.permute(0, 2, 3, 1, 4), rpb, kernel_size, dilation)
    return out.permute(0, 3, 1, 2, 4)


def natten2dav(attn, value, kernel_size, dilation):
    """attn ``[B, H, Hh, Hw, Kh*Kw]``, value ``[B, H, Hh, Hw, D]`` -> ``[B, H, Hh, Hw, D]``."""
    if attn.ndim != 5 or value.ndim != 5:
        raise ValueError("natten2dav expects attn [B,H,Hh,Hw,K] and value [B,H,Hh,Hw,D].")
    out = F.na2d_av(attn.permute(0, 2, 3, 1, 4), value.permute(0, 2, 3, 1, 4), kernel_size, dilation)
    return out.permute(0, 3, 1, 2, 4)


__all__ = ["natten1dqkrpb", "natten1dav", "natten2dqkrpb", "natten2dav"]
