"""ctypes binding of ``libnatten_b200.so`` (declared in ``include/natten_b200.h``).

This is the only place the Python package touches native code.  There is no
CPU or PyTorch fallback: if the library is missing, importing an op raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence, Tuple

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libnatten_b200.so")

F32, F16, BF16, F64 = 0, 1, 2, 3
FLAG_FORCE_SIMT, FLAG_FORCE_TC = 1, 2
OP_FUSED_FWD, OP_FUSED_BWD = 0, 1
PATH_NAMES = {0: "none", 1: "simt", 2: "tcgen05"}

EXPORTS = (
    "natten_fused_fwd", "natten_fused_bwd", "natten_workspace_bytes", "natten_qk_fwd",
    "natten_qk_bwd", "natten_qk_rpb_fwd", "natten_qk_rpb_bwd", "natten_av_fwd", "natten_av_bwd", "natten_strerror",
    "natten_abi_version", "natten_last_path", "natten_launch_count", "natten_device_status",
    "natten_clear_status", "natten_status_async", "natten_debug_wait",
    "natten_fused_bwd_static", "natten_static_scratch_bytes",
)

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.float64: F64}


class Params(ctypes.Structure):
    """Mirror of ``natten_params_t``."""
    _fields_ = [
        ("rank", ctypes.c_int32), ("dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32), ("heads_q", ctypes.c_int32), ("heads_kv", ctypes.c_int32),
        ("dim", ctypes.c_int32), ("dim_v", ctypes.c_int32),
        ("extent", ctypes.c_int32 * 3), ("kernel", ctypes.c_int32 * 3),
        ("dilation", ctypes.c_int32 * 3), ("stride", ctypes.c_int32 * 3),
        ("causal", ctypes.c_int32 * 3),
        ("n_extra", ctypes.c_int32), ("has_scale", ctypes.c_int32), ("flags", ctypes.c_int32),
        ("scale", ctypes.c_double),
        ("q_stride", ctypes.c_int64 * 3), ("k_stride", ctypes.c_int64 * 3),
        ("v_stride", ctypes.c_int64 * 3),
        ("extents", ctypes.c_void_p),
    ]


_lib = None
_force_flags = 0


def lib():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m natten_mps_b200._build` "
                "(there is no fallback implementation)")
        L = ctypes.CDLL(LIB_PATH)
        vp = ctypes.c_void_p
        pp = ctypes.POINTER(Params)
        L.natten_fused_fwd.argtypes = [pp] + [vp] * 8
        L.natten_fused_bwd.argtypes = [pp] + [vp] * 15 + [ctypes.c_size_t, vp]
        L.natten_fused_bwd_static.argtypes = [pp] + [vp] * 15
        L.natten_static_scratch_bytes.restype = ctypes.c_size_t
        L.natten_workspace_bytes.argtypes = [pp, ctypes.c_int]
        L.natten_workspace_bytes.restype = ctypes.c_size_t
        L.natten_qk_fwd.argtypes = [pp] + [vp] * 4
        L.natten_qk_bwd.argtypes = [pp] + [vp] * 6
        L.natten_qk_rpb_fwd.argtypes = [pp] + [vp] * 5
        L.natten_qk_rpb_bwd.argtypes = [pp] + [vp] * 7
        L.natten_av_fwd.argtypes = [pp] + [vp] * 4
        L.natten_av_bwd.argtypes = [pp] + [vp] * 6
        L.natten_strerror.argtypes = [ctypes.c_int]
        L.natten_strerror.restype = ctypes.c_char_p
        L.natten_launch_count.restype = ctypes.c_ulonglong
        L.natten_status_async.argtypes = [vp, vp]
        L.natten_debug_wait.argtypes = [ctypes.c_longlong, ctypes.c_int]
        L.natten_debug_wait.restype = None
        for name in EXPORTS:
            getattr(L, name)
        _lib = L
    return _lib


def set_force(path: Optional[str]) -> None:
    """Testing aid: force ``"simt"`` or ``"tc"`` kernels (``None`` = automatic)."""
    global _force_flags
    _force_flags = {None: 0, "auto": 0, "simt": FLAG_FORCE_SIMT, "tc": FLAG_FORCE_TC}[path]


def last_path() -> str:
    return PATH_NAMES[lib().natten_last_path()]


def device_status() -> int:
    """0 when no kernel ever gave up on a bounded wait (synchronises the device)."""
    return int(lib().natten_device_status())


def clear_status() -> None:
    """Reset the current device's status word after a kernel gave up on a wait (synchronises)."""
    rc = int(lib().natten_clear_status())
    for w in _status_words.values():
        w.zero_()
    if rc:
        raise RuntimeError(f"natten_clear_status: CUDA error {rc}")


# One pinned host word per device.  After every launch the library copies the device's status
# word into it on the launching stream; the word is looked at (a plain host read) at the next
# call and by ``poll_status``, so a kernel that gave up surfaces as a RuntimeError instead of
# silently empty results.
_status_words = {}


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32).pin_memory()
        _status_words[idx] = w
    return w


def poll_status(device: torch.device) -> None:
    """Raise if a kernel on ``device`` reported a timed-out wait (no synchronisation: sees what
    the stream has copied back so far)."""
    if int(_status_word(device)[0]) != 0:
        raise RuntimeError(
            "natten_b200: a tensor-core kernel gave up on a bounded wait (results since then are "
            "invalid); call natten_mps_b200._cabi.clear_status() to re-arm the device")


def track_status(t: torch.Tensor) -> None:
    """Enqueue the status copy behind the kernels just launched on ``t``'s current stream."""
    w = _status_word(t.device)
    with torch.cuda.device(t.device):
        lib().natten_status_async(ctypes.c_void_p(w.data_ptr()), stream_of(t))


def launch_count() -> int:
    return int(lib().natten_launch_count())


def check(code: int, what: str) -> None:
    if code == 0:
        return
    msg = f"{what}: {lib().natten_strerror(code).decode()} (code {code})"
    if code == -1:
        raise ValueError(msg)
    if code == -2:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)


def token_strides(t: torch.Tensor, rank: int) -> Optional[Tuple[int, int, int]]:
    """(batch, token, head) element strides if the spatial axes collapse into one
    token axis and the channel axis is contiguous; otherwise ``None``."""
    st, sz = t.stride(), t.shape
    if sz[-1] != 1 and st[-1] != 1:
        return None
    tok = st[rank]
    for a in range(rank - 1, 0, -1):
        if sz[a + 1] != 1 and st[a] != st[a + 1] * sz[a + 1]:
            return None
    if any(s < 0 for s in st):
        return None
    return (st[0], tok, st[-2])


def as_strided_input(t: torch.Tensor, rank: int) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    s = token_strides(t, rank)
    if s is None:
        t = t.contiguous()
        s = token_strides(t, rank)
    return t, s


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_of(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def make_params(rank: int, dtype: torch.dtype, batch: int, heads_q: int, heads_kv: int, dim: int,
                dim_v: int, spatial: Sequence[int], kernel_size: Sequence[int],
                stride: Sequence[int], dilation: Sequence[int], is_causal: Sequence[bool],
                scale: Optional[float], n_extra: int = 0,
                q_stride=(0, 0, 0), k_stride=(0, 0, 0), v_stride=(0, 0, 0),
                extents: Optional[torch.Tensor] = None) -> Params:
    if dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {dtype}; expected float32, float16, bfloat16 or float64")
    p = Params()
    p.rank, p.dtype = rank, _DTYPES[dtype]
    p.batch, p.heads_q, p.heads_kv, p.dim, p.dim_v = batch, heads_q, heads_kv, dim, dim_v
    for a in range(3):
        on = a < rank
        p.extent[a] = int(spatial[a]) if on else 1
        p.kernel[a] = int(kernel_size[a]) if on else 1
        p.dilation[a] = int(dilation[a]) if on else 1
        p.stride[a] = int(stride[a]) if on else 1
        p.causal[a] = int(bool(is_causal[a])) if on else 0
    p.n_extra = int(n_extra)
    p.has_scale = int(scale is not None)
    p.scale = float(scale) if scale is not None else 1.0
    p.flags = _force_flags
    for i in range(3):
        p.q_stride[i], p.k_stride[i], p.v_stride[i] = int(q_stride[i]), int(k_stride[i]), int(v_stride[i])
    p.extents = extents.data_ptr() if extents is not None else None
    return p
