"""Neighbourhood attention for NVIDIA B200 -- the natten-mps API on one CUDA path.

``import natten_mps_b200`` does not import torch; public names are resolved on
first access (the reference does the same, ``src/natten_mps/__init__.py:41-73``).
"""
from __future__ import annotations

from .version import __version__

_LAZY = {
    **{n: "functional" for n in (
        "na1d", "na2d", "na3d", "na1d_qk", "na1d_av", "na2d_qk", "na2d_av", "na3d_qk", "na3d_av",
        "na1d_varlen", "na2d_varlen", "na3d_varlen")},
    "merge_attentions": "merge",
    "NeighborhoodAttention1D": "nn", "NeighborhoodAttention2D": "nn", "NeighborhoodAttention3D": "nn",
    "get_support_matrix": "support_matrix",
    "HostStep": "host_step",
}

__all__ = sorted(list(_LAZY) + ["has_cuda", "get_backend", "set_backend", "__version__"])


def __getattr__(name: str):
    target = _LAZY.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    import importlib
    return getattr(importlib.import_module(f"{__name__}.{target}"), name)


def __dir__():
    return __all__


def has_cuda() -> bool:
    """True when a CUDA device is visible and the native library has been built."""
    from . import ops
    return ops.is_available()


def get_backend() -> str:
    from . import ops
    return ops.get_backend()


def set_backend(name: str) -> None:
    from . import ops
    ops.set_backend(name)
