"""Capability matrix (same shape as the reference's ``get_support_matrix``,
``src/natten_mps/support_matrix.py:8-37``, with a single ``cuda`` tier)."""
from __future__ import annotations


def get_support_matrix() -> dict:
    from . import ops
    yes = {"na1d": True, "na2d": True, "na3d": True}
    return {
        "cuda": {
            "available": ops.is_available(),
            "forward": {**yes, "split_qk_av": True},
            "backward": {**yes, "split_qk_av": True},
            "varlen": dict(yes),
            "fusion": dict(yes),
            "constraints": [
                "Requires an NVIDIA B200 (sm_100a) and the in-tree libnatten_b200.so.",
                "float32, float16, bfloat16 and float64; head dim <= 256.",
                "Causal masking per axis, stride, dilation, non-uniform kernels, GQA/MQA, "
                "additional key/value tokens and per-sample extents are kernel arguments.",
                "No CPU fallback: CPU tensors are rejected.",
            ],
        }
    }
