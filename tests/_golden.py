"""Loader for the fixtures written by tests/golden/make_golden.py."""
import json
import os

import numpy as np

_HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
_npz = None
_manifest = None


def manifest():
    global _manifest
    if _manifest is None:
        with open(os.path.join(_HERE, "golden.json")) as f:
            _manifest = json.load(f)
    return _manifest


def arrays(name):
    """All arrays of one case as a dict (float64 / int)."""
    global _npz
    if _npz is None:
        _npz = np.load(os.path.join(_HERE, "golden.npz"))
    out = {}
    for key in _npz.files:
        if key.startswith(name + "/"):
            a = _npz[key]
            out[key.split("/", 1)[1]] = a.astype(np.float64) if a.dtype.kind == "f" else a
    return out


def kw(case):
    """kwargs of a case with JSON lists turned back into tuples."""
    return {k: (tuple(v) if isinstance(v, list) else v) for k, v in case["kwargs"].items()}


def fused_cases():
    return manifest()["fused"]


def split_cases():
    return manifest()["split"]


def module_cases():
    return manifest().get("modules", [])


def rpb_cases():
    return manifest().get("rpb", [])


def pb_rows():
    """Yield (index, length, kernel, dilation, pb_start) in the order of the window table."""
    vals = arrays("window")["pb_start"]
    n = 0
    for L in range(1, 41):
        for K in range(1, 12):
            for dil in range(1, 5):
                if K * dil > L:
                    continue
                for i in range(L):
                    yield i, L, K, dil, int(vals[n])
                    n += 1
    assert n == len(vals)


def varlen_cases():
    return manifest()["varlen"]


def window_rows():
    """Yield (index, length, kernel, dilation, start) in the fixture's order."""
    starts = arrays("window")["start"]
    n = 0
    for L in range(1, 41):
        for K in range(1, 12):
            for dil in range(1, 5):
                if K * dil > L:
                    continue
                for i in range(L):
                    yield i, L, K, dil, int(starts[n])
                    n += 1
    assert n == len(starts)
