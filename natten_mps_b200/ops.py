"""The reference's backend protocol, served by the CUDA library.

``src/natten_mps/_core/ops.py:90-152`` defines nine functions per backend
(``na{R}d_forward``, ``na{R}d_qk_forward``, ``na{R}d_av_forward``,
``na{R}d_qk_backward``, ``na{R}d_av_backward``).  This module offers the same
names and argument orders -- note fused takes ``(kernel_size, stride, dilation)``
while the split ops take ``(kernel_size, dilation, stride)`` -- plus
``na{R}d_forward_with_lse`` and ``na{R}d_fused_backward`` that the reference's
accelerated backend adds (``src/natten_mps/autograd/_factory.py:33-41, 63-74``).
There is one backend, ``"cuda"``; ``set_backend`` only accepts it (or ``"auto"``).
"""
from __future__ import annotations

from typing import Optional

from . import _backend

_BACKEND = "cuda"


def get_backend() -> str:
    return _BACKEND


def set_backend(name: str) -> None:
    if name not in ("auto", "cuda"):
        raise NotImplementedError(
            f"backend {name!r} is not available: this package has a single CUDA path "
            "(choose 'cuda' or 'auto')")


def is_available() -> bool:
    import torch
    from . import _cabi
    import os
    return torch.cuda.is_available() and os.path.exists(_cabi.LIB_PATH)


def _scale_of(q, scale: Optional[float]) -> float:
    return float(q.shape[-1] ** -0.5 if scale is None else scale)


def _make(rank: int):
    def forward(q, k, v, kernel_size, stride, dilation, is_causal, scale):
        return _backend.fused_forward(q, k, v, tuple(kernel_size), tuple(stride), tuple(dilation),
                                      tuple(is_causal), _scale_of(q, scale))[0]

    def forward_with_lse(q, k, v, kernel_size, stride, dilation, is_causal, scale):
        return _backend.fused_forward(q, k, v, tuple(kernel_size), tuple(stride), tuple(dilation),
                                      tuple(is_causal), _scale_of(q, scale))

    def fused_backward(q, k, v, out, lse, grad_out, kernel_size, stride, dilation, is_causal, scale):
        return _backend.fused_backward(q, k, v, out, lse, grad_out, tuple(kernel_size), tuple(stride),
                                       tuple(dilation), tuple(is_causal), _scale_of(q, scale))[:3]

    def qk_forward(q, k, kernel_size, dilation, stride=(1,) * rank, is_causal=(False,) * rank, scale=None):
        return _backend.qk_forward(q, k, tuple(kernel_size), tuple(dilation), tuple(stride),
                                   tuple(is_causal), scale)

    def av_forward(attn, v, kernel_size, dilation, stride=(1,) * rank, is_causal=(False,) * rank):
        return _backend.av_forward(attn, v, tuple(kernel_size), tuple(dilation), tuple(stride),
                                   tuple(is_causal))

    def qk_backward(d_attn, q, k, kernel_size, dilation, stride=(1,) * rank, is_causal=(False,) * rank,
                    scale=None):
        return _backend.qk_backward(d_attn, q, k, tuple(kernel_size), tuple(dilation), tuple(stride),
                                    tuple(is_causal), scale)

    def av_backward(d_out, attn, v, kernel_size, dilation, stride=(1,) * rank, is_causal=(False,) * rank):
        return _backend.av_backward(d_out, attn, v, tuple(kernel_size), tuple(dilation), tuple(stride),
                                    tuple(is_causal))

    g = globals()
    for name, fn in (("forward", forward), ("forward_with_lse", forward_with_lse),
                     ("fused_backward", fused_backward), ("qk_forward", qk_forward),
                     ("av_forward", av_forward), ("qk_backward", qk_backward),
                     ("av_backward", av_backward)):
        fn.__name__ = f"na{rank}d_{name}"
        g[fn.__name__] = fn


for _r in (1, 2, 3):
    _make(_r)
