"""``NeighborhoodAttention{1,2,3}D`` modules: qkv projection -> neighbourhood
attention -> output projection.

Constructor arguments, parameter names (``qkv`` or ``q_proj`` + ``kv_proj``,
``proj``) and ``forward(x, sizes=None)`` follow the reference's
``src/natten_mps/nn/na1d.py:11-130`` (and ``na2d.py`` / ``na3d.py``), so
``state_dict``s interchange.  The q/k/v handed to the kernels are strided views
of the projection output; the C ABI takes their strides, nothing is copied.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from .. import functional as F
from ..utils.params import normalize_tuple_param

_FUSED = {1: F.na1d, 2: F.na2d, 3: F.na3d}
_QK = {1: F.na1d_qk, 2: F.na2d_qk, 3: F.na3d_qk}
_AV = {1: F.na1d_av, 2: F.na2d_av, 3: F.na3d_av}
_VARLEN = {1: F.na1d_varlen, 2: F.na2d_varlen, 3: F.na3d_varlen}
_IN_LAYOUT = {1: "[B, L, C]", 2: "[B, H, W, C]", 3: "[B, D, H, W, C]"}


class _NeighborhoodAttention(torch.nn.Module):
    rank = 0

    def __init__(self, embed_dim: int, num_heads: int, kernel_size: Union[int, Tuple[int, ...]],
                 stride: Union[int, Tuple[int, ...]] = 1, dilation: Union[int, Tuple[int, ...]] = 1,
                 is_causal: Union[bool, Tuple[bool, ...]] = False,
                 num_kv_heads: Optional[int] = None, qkv_bias: bool = True,
                 qk_scale: Optional[float] = None, attn_drop: float = 0.0, proj_drop: float = 0.0):
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError("embed_dim must be divisible by num_heads")
        r = self.rank
        self.embed_dim, self.num_heads = int(embed_dim), int(num_heads)
        self.head_dim = self.embed_dim // self.num_heads
        self.num_kv_heads = self.num_heads if num_kv_heads is None else int(num_kv_heads)
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(
                f"num_heads ({self.num_heads}) must be divisible by num_kv_heads ({self.num_kv_heads})")
        self.kernel_size = normalize_tuple_param(kernel_size, r, "kernel_size")
        self.stride = normalize_tuple_param(stride, r, "stride")
        self.dilation = normalize_tuple_param(dilation, r, "dilation")
        self.is_causal = tuple(bool(v) for v in normalize_tuple_param(is_causal, r, "is_causal"))
        self.scale = self.head_dim ** -0.5 if qk_scale is None else float(qk_scale)
        self._use_gqa = self.num_kv_heads != self.num_heads
        if self._use_gqa:
            self.q_proj = torch.nn.Linear(self.embed_dim, self.num_heads * self.head_dim, bias=qkv_bias)
            self.kv_proj = torch.nn.Linear(self.embed_dim, 2 * self.num_kv_heads * self.head_dim, bias=qkv_bias)
        else:
            self.qkv = torch.nn.Linear(self.embed_dim, 3 * self.embed_dim, bias=qkv_bias)
        self.attn_drop_p = float(attn_drop)
        self.attn_drop = torch.nn.Dropout(attn_drop)
        self.proj = torch.nn.Linear(self.embed_dim, self.embed_dim)
        self.proj_drop = torch.nn.Dropout(proj_drop)

    def _project(self, x):
        lead = x.shape[:-1]
        if self._use_gqa:
            q = self.q_proj(x).reshape(*lead, self.num_heads, self.head_dim)
            kv = self.kv_proj(x).reshape(*lead, 2, self.num_kv_heads, self.head_dim)
            k, v = kv.unbind(dim=-3)
        else:
            q, k, v = self.qkv(x).reshape(*lead, 3, self.num_heads, self.head_dim).unbind(dim=-3)
        return q, k, v

    def forward(self, x: torch.Tensor, sizes: Optional[torch.Tensor] = None) -> torch.Tensor:
        r = self.rank
        if x.ndim != r + 2:
            raise ValueError(f"{type(self).__name__} expects input shape {_IN_LAYOUT[r]}.")
        if x.shape[-1] != self.embed_dim:
            raise ValueError(
                f"Input channel dim ({x.shape[-1]}) must equal embed_dim ({self.embed_dim}).")
        q, k, v = self._project(x)
        if sizes is not None:
            out = _VARLEN[r](q, k, v, sizes, kernel_size=self.kernel_size, dilation=self.dilation,
                             scale=self.scale)
        elif self.attn_drop_p > 0.0:
            # Same behaviour as the reference's dropout branch (nn/na1d.py:108-114): the
            # split ops take matching head counts, logits are left unscaled unless a
            # custom qk_scale was given, and stride / causal flags are not applied.
            if self._use_gqa:
                rep = self.num_heads // self.num_kv_heads
                k, v = k.repeat_interleave(rep, dim=-2), v.repeat_interleave(rep, dim=-2)
            logits = _QK[r](q, k, kernel_size=self.kernel_size, dilation=self.dilation)
            default_scale = self.head_dim ** -0.5
            if self.scale != default_scale:
                logits = logits * (self.scale / default_scale)
            attn = self.attn_drop(torch.softmax(logits, dim=-1))
            out = _AV[r](attn, v, kernel_size=self.kernel_size, dilation=self.dilation)
        else:
            out = _FUSED[r](q, k, v, kernel_size=self.kernel_size, stride=self.stride,
                            dilation=self.dilation, is_causal=self.is_causal, scale=self.scale)
        out = out.reshape(*out.shape[:-2], self.embed_dim)
        return self.proj_drop(self.proj(out))


class NeighborhoodAttention1D(_NeighborhoodAttention):
    """1-D module; ``forward(x [B, L, C], seq_lens=None)``."""
    rank = 1

    def forward(self, x, seq_lens=None):  # noqa: D102
        return super().forward(x, seq_lens)


class NeighborhoodAttention2D(_NeighborhoodAttention):
    """2-D module; ``forward(x [B, H, W, C], spatial_sizes=None)``."""
    rank = 2

    def forward(self, x, spatial_sizes=None):  # noqa: D102
        return super().forward(x, spatial_sizes)


class NeighborhoodAttention3D(_NeighborhoodAttention):
    """3-D module; ``forward(x [B, D, H, W, C], spatial_sizes=None)``."""
    rank = 3

    def forward(self, x, spatial_sizes=None):  # noqa: D102
        return super().forward(x, spatial_sizes)
