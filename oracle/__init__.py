"""TEST INFRASTRUCTURE ONLY -- numpy front end of the CPU oracle.

``oracle/natten_oracle.c`` restates the reference's pure backend
(``src/natten_mps/_core/pure.py``, ``src/natten_mps/utils/window.py``) as plain
C loops.  This module builds it with gcc on first use, binds it with ctypes and
exposes array-in / array-out helpers.  Only the test-suite, the smoke check and
the CPU-baseline leg of the benchmark may import it; the shipped package never
does and has no CPU fallback.

Arrays are float32 or float64 (the oracle computes in that precision),
contiguous and heads-last: ``q [B, *L, Hq, D]``, ``k [B, *L, Hkv, D]``,
``v [B, *L, Hkv, Dv]``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "natten_oracle.c")
_LIB = os.path.join(_HERE, "libnatten_oracle.so")


class _Params(ctypes.Structure):
    _fields_ = [
        ("rank", ctypes.c_int),
        ("B", ctypes.c_int), ("Hq", ctypes.c_int), ("Hkv", ctypes.c_int),
        ("D", ctypes.c_int), ("Dv", ctypes.c_int),
        ("L", ctypes.c_int * 3),
        ("K", ctypes.c_int * 3), ("dil", ctypes.c_int * 3),
        ("stride", ctypes.c_int * 3), ("causal", ctypes.c_int * 3),
        ("has_scale", ctypes.c_int),
        ("n_extra", ctypes.c_int),
        ("scale", ctypes.c_double),
        ("extents", ctypes.c_void_p),
    ]


def build(force: bool = False) -> str:
    """Compile the C oracle next to its source (gcc, OpenMP)."""
    body = os.path.join(_HERE, "natten_oracle_body.inc")
    stale = (not os.path.exists(_LIB)) or any(
        os.path.getmtime(p) > os.path.getmtime(_LIB) for p in (_SRC, body) if os.path.exists(p)
    )
    if force or stale:
        subprocess.check_call(
            ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", _SRC, "-o", _LIB, "-lm"]
        )
    return _LIB


_lib = None


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.ora_window_start.restype = ctypes.c_int
        _lib.ora_window_start.argtypes = [ctypes.c_int] * 4
    return _lib


def pb_start(index: int, length: int, kernel_size: int, dilation: int) -> int:
    """``get_pb_start`` of ``utils/window.py:119-135``."""
    lib = _load()
    lib.ora_pb_start.restype = ctypes.c_int
    lib.ora_pb_start.argtypes = [ctypes.c_int] * 4
    return int(lib.ora_pb_start(index, length, kernel_size, dilation))


def window_start(index: int, length: int, kernel_size: int, dilation: int) -> int:
    """``get_window_start`` of ``utils/window.py:91-111``."""
    return int(_load().ora_window_start(index, length, kernel_size, dilation))


def _tup(x, rank, cast=int):
    if isinstance(x, (int, bool, np.integer)):
        return (cast(x),) * rank
    x = tuple(cast(v) for v in x)
    assert len(x) == rank
    return x


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


class _Call:
    """Collects geometry for one oracle call and keeps arrays alive."""

    def __init__(self, rank, q_shape, hkv, dv, kernel_size, stride, dilation, is_causal,
                 scale, has_scale, extents, n_extra):
        self.rank = rank
        spatial = tuple(int(s) for s in q_shape[1:1 + rank])
        p = _Params()
        p.rank = rank
        p.B, p.Hq, p.D = int(q_shape[0]), int(q_shape[-2]), int(q_shape[-1])
        p.Hkv, p.Dv = int(hkv), int(dv)
        ks, st = _tup(kernel_size, rank), _tup(stride, rank)
        dil, ca = _tup(dilation, rank), _tup(is_causal, rank, bool)
        for a in range(3):
            p.L[a] = spatial[a] if a < rank else 1
            p.K[a] = ks[a] if a < rank else 1
            p.dil[a] = dil[a] if a < rank else 1
            p.stride[a] = st[a] if a < rank else 1
            p.causal[a] = int(ca[a]) if a < rank else 0
        p.has_scale = int(has_scale)
        p.n_extra = int(n_extra)
        p.scale = float(scale)
        self._ext = None
        if extents is not None:
            self._ext = np.ascontiguousarray(np.asarray(extents).reshape(p.B, rank), dtype=np.int32)
            p.extents = self._ext.ctypes.data
        self.p = p
        self.spatial = spatial
        self.out_spatial = tuple((spatial[a] + st[a] - 1) // st[a] for a in range(rank))
        self.ktot = int(np.prod(ks))


def _prep(dtype, *arrays):
    out = []
    for a in arrays:
        out.append(None if a is None else np.ascontiguousarray(a, dtype=dtype))
    return out


def _suffix(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "_f32"
    if dtype == np.float64:
        return "_f64"
    raise TypeError("the oracle computes in float32 or float64")


def na_forward(q, k, v, kernel_size, stride=1, dilation=1, is_causal=False, scale=None,
               additional_keys=None, additional_values=None, extents=None, dtype=np.float64):
    """Fused forward -> ``(out, lse)`` (``_core/pure.py:146-220, 397-433``)."""
    rank = q.ndim - 3
    q, k, v, ek, ev = _prep(dtype, q, k, v, additional_keys, additional_values)
    sc = q.shape[-1] ** -0.5 if scale is None else float(scale)
    n_extra = 0 if ek is None else ek.shape[1]
    c = _Call(rank, q.shape, k.shape[-2], v.shape[-1], kernel_size, stride, dilation, is_causal,
              sc, 1, extents, n_extra)
    out = np.empty((q.shape[0],) + c.out_spatial + (q.shape[-2], v.shape[-1]), dtype=dtype)
    lse = np.empty((q.shape[0],) + c.out_spatial + (q.shape[-2],), dtype=dtype)
    fn = getattr(_load(), "ora_fwd" + _suffix(dtype))
    fn.restype = None
    fn(ctypes.byref(c.p), _ptr(q), _ptr(k), _ptr(v), _ptr(ek), _ptr(ev), _ptr(out), _ptr(lse))
    return out, lse


def na_backward(q, k, v, out, lse, dout, kernel_size, stride=1, dilation=1, is_causal=False,
                scale=None, additional_keys=None, additional_values=None, extents=None,
                dlse=None, dtype=np.float64):
    """Fused backward -> ``(dq, dk, dv, d_extra_k, d_extra_v)``."""
    rank = q.ndim - 3
    q, k, v, ek, ev, out, lse, dout, dlse = _prep(
        dtype, q, k, v, additional_keys, additional_values, out, lse, dout, dlse)
    sc = q.shape[-1] ** -0.5 if scale is None else float(scale)
    n_extra = 0 if ek is None else ek.shape[1]
    c = _Call(rank, q.shape, k.shape[-2], v.shape[-1], kernel_size, stride, dilation, is_causal,
              sc, 1, extents, n_extra)
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    dek = None if ek is None else np.empty_like(ek)
    dev = None if ev is None else np.empty_like(ev)
    fn = getattr(_load(), "ora_bwd" + _suffix(dtype))
    fn.restype = None
    fn(ctypes.byref(c.p), _ptr(q), _ptr(k), _ptr(v), _ptr(ek), _ptr(ev), _ptr(out), _ptr(lse),
       _ptr(dout), _ptr(dlse), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dek), _ptr(dev))
    return dq, dk, dv, dek, dev


def na_qk(q, k, kernel_size, dilation=1, stride=1, is_causal=False, scale=None, dtype=np.float64):
    """Split QK forward -> logits (``_core/pure.py:223-254, 294-332, 436-471``)."""
    rank = q.ndim - 3
    q, k = _prep(dtype, q, k)
    c = _Call(rank, q.shape, k.shape[-2], q.shape[-1], kernel_size, stride, dilation, is_causal,
              1.0 if scale is None else scale, scale is not None, None, 0)
    logits = np.empty((q.shape[0],) + c.out_spatial + (q.shape[-2], c.ktot), dtype=dtype)
    fn = getattr(_load(), "ora_qk_fwd" + _suffix(dtype))
    fn.restype = None
    fn(ctypes.byref(c.p), _ptr(q), _ptr(k), _ptr(logits))
    return logits


def na_qk_backward(q, k, dlogits, kernel_size, dilation=1, stride=1, is_causal=False, scale=None,
                   dtype=np.float64):
    """Split QK backward -> ``(dq, dk)``."""
    rank = q.ndim - 3
    q, k, dlogits = _prep(dtype, q, k, dlogits)
    c = _Call(rank, q.shape, k.shape[-2], q.shape[-1], kernel_size, stride, dilation, is_causal,
              1.0 if scale is None else scale, scale is not None, None, 0)
    dq, dk = np.empty_like(q), np.empty_like(k)
    fn = getattr(_load(), "ora_qk_bwd" + _suffix(dtype))
    fn.restype = None
    fn(ctypes.byref(c.p), _ptr(q), _ptr(k), _ptr(dlogits), _ptr(dq), _ptr(dk))
    return dq, dk


def _av_call(attn, v, kernel_size, dilation, stride, is_causal):
    rank = v.ndim - 3
    # geometry is described through a query-shaped tuple: [B, *L, Hq, D]
    q_shape = (v.shape[0],) + tuple(v.shape[1:1 + rank]) + (attn.shape[-2], v.shape[-1])
    return _Call(rank, q_shape, v.shape[-2], v.shape[-1], kernel_size, stride, dilation,
                 is_causal, 1.0, 0, None, 0)


def na_av(attn, v, kernel_size, dilation=1, stride=1, is_causal=False, dtype=np.float64):
    """Split AV forward (``_core/pure.py:257-291, 520-565, 474-517``)."""
    attn, v = _prep(dtype, attn, v)
    c = _av_call(attn, v, kernel_size, dilation, stride, is_causal)
    assert tuple(attn.shape[1:-2]) == c.out_spatial and attn.shape[-1] == c.ktot
    out = np.empty((v.shape[0],) + c.out_spatial + (attn.shape[-2], v.shape[-1]), dtype=dtype)
    fn = getattr(_load(), "ora_av_fwd" + _suffix(dtype))
    fn.restype = None
    fn(ctypes.byref(c.p), _ptr(attn), _ptr(v), _ptr(out))
    return out


def na_av_backward(attn, v, dout, kernel_size, dilation=1, stride=1, is_causal=False,
                   dtype=np.float64):
    """Split AV backward -> ``(dattn, dv)``."""
    attn, v, dout = _prep(dtype, attn, v, dout)
    c = _av_call(attn, v, kernel_size, dilation, stride, is_causal)
    dattn, dv = np.empty_like(attn), np.empty_like(v)
    fn = getattr(_load(), "ora_av_bwd" + _suffix(dtype))
    fn.restype = None
    fn(ctypes.byref(c.p), _ptr(attn), _ptr(v), _ptr(dout), _ptr(dattn), _ptr(dv))
    return dattn, dv


def na_qk_rpb(q, k, rpb, kernel_size, dilation=1, scale=None, dtype=np.float64):
    """Split QK plus relative position bias (``compat/v014.py:66-183``, heads-last layout)."""
    logits = na_qk(q, k, kernel_size, dilation=dilation, scale=scale, dtype=dtype)
    rank = q.ndim - 3
    if any(int(x) % 2 == 0 for x in np.broadcast_to(np.asarray(kernel_size), (rank,))):
        raise ValueError("relative position bias needs odd kernel sizes (the lookup runs past the table otherwise)")
    (rpb,) = _prep(dtype, rpb)
    c = _Call(rank, q.shape, k.shape[-2], q.shape[-1], kernel_size, 1, dilation, False, 1.0, 0, None, 0)
    fn = getattr(_load(), "ora_rpb_add" + _suffix(dtype))
    fn.restype = None
    fn(ctypes.byref(c.p), _ptr(rpb), _ptr(logits))
    return logits


def na_qk_rpb_backward(q, k, rpb, dlogits, kernel_size, dilation=1, scale=None, dtype=np.float64):
    """-> ``(dq, dk, d_rpb)``."""
    dq, dk = na_qk_backward(q, k, dlogits, kernel_size, dilation=dilation, scale=scale, dtype=dtype)
    rank = q.ndim - 3
    (dl,) = _prep(dtype, dlogits)
    c = _Call(rank, q.shape, k.shape[-2], q.shape[-1], kernel_size, 1, dilation, False, 1.0, 0, None, 0)
    drpb = np.empty(np.asarray(rpb).shape, dtype=dtype)
    fn = getattr(_load(), "ora_rpb_grad" + _suffix(dtype))
    fn.restype = None
    fn(ctypes.byref(c.p), _ptr(dl), _ptr(drpb))
    return dq, dk, drpb
