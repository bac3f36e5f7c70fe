"""The CPU oracle against the outputs of the reference itself (tests/golden)."""
import numpy as np
import pytest

import oracle
from tests import _golden as G

TOL = 1e-10  # float64 oracle vs float64 reference


def _close(a, b, tol=TOL):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape
    fa, fb = np.isfinite(a), np.isfinite(b)
    assert np.array_equal(fa, fb)
    assert np.array_equal(a[~fa], b[~fb])          # the -inf pattern matches exactly
    scale = max(1.0, float(np.abs(b[fb]).max()) if fb.any() else 1.0)
    assert float(np.abs(a[fa] - b[fb]).max() if fa.any() else 0.0) <= tol * scale


def test_window_start_table():
    n = 0
    for i, L, K, dil, start in G.window_rows():
        assert oracle.window_start(i, L, K, dil) == start, (i, L, K, dil)
        n += 1
    assert n == G.manifest()["window"]["rows"]


@pytest.mark.parametrize("case", G.fused_cases(), ids=lambda c: c["name"])
def test_fused_forward_backward(case):
    a = G.arrays(case["name"])
    kw = G.kw(case)
    want_lse = kw.pop("return_lse", False)
    # the reference merges the additional-token attention in float32 (merge.py:26-33)
    tol = 2e-6 if case["n_extra"] else TOL
    out, lse = oracle.na_forward(a["q"], a["k"], a["v"], additional_keys=a.get("ek"),
                                 additional_values=a.get("ev"), **kw)
    _close(out, a["out"], tol)
    if want_lse:
        _close(lse, a["lse"], tol)
    grads = oracle.na_backward(a["q"], a["k"], a["v"], out, lse, a["gout"],
                               additional_keys=a.get("ek"), additional_values=a.get("ev"),
                               dlse=a.get("glse"), **kw)
    for name, g in zip(["dq", "dk", "dv", "dek", "dev"], grads):
        if name in a:
            _close(g, a[name], tol)


@pytest.mark.parametrize("case", G.split_cases(), ids=lambda c: c["name"])
def test_split_ops(case):
    a = G.arrays(case["name"])
    kw = G.kw(case)
    _close(oracle.na_qk(a["q"], a["k"], **kw), a["logits"])
    dq, dk = oracle.na_qk_backward(a["q"], a["k"], a["glog"], **kw)
    _close(dq, a["dq"])
    _close(dk, a["dk"])
    kw.pop("scale", None)
    _close(oracle.na_av(a["attn"], a["v"], **kw), a["out"])
    dattn, dv = oracle.na_av_backward(a["attn"], a["v"], a["gout"], **kw)
    _close(dattn, a["dattn"])
    _close(dv, a["dv"])


@pytest.mark.parametrize("case", G.varlen_cases(), ids=lambda c: c["name"])
def test_varlen(case):
    a = G.arrays(case["name"])
    kw = G.kw(case)
    out, lse = oracle.na_forward(a["q"], a["k"], a["v"], extents=case["sizes"], **kw)
    _close(out, a["out"])
    dq, dk, dv, _, _ = oracle.na_backward(a["q"], a["k"], a["v"], out, lse, a["gout"],
                                          extents=case["sizes"], **kw)
    _close(dq, a["dq"])
    _close(dk, a["dk"])
    _close(dv, a["dv"])


def test_float32_oracle_tracks_float64():
    a = G.arrays("na2d_basic")
    o64, _ = oracle.na_forward(a["q"], a["k"], a["v"], kernel_size=(3, 5))
    o32, _ = oracle.na_forward(a["q"], a["k"], a["v"], kernel_size=(3, 5), dtype=np.float32)
    assert np.abs(o64 - o32).max() < 1e-5


def test_pb_start_matches_reference_table():
    from natten_mps_b200.utils import get_pb_start
    for i, L, K, dil, want in G.pb_rows():
        assert oracle.pb_start(i, L, K, dil) == want
        assert get_pb_start(i, L, K, dil) == want


@pytest.mark.parametrize("case", G.rpb_cases(), ids=lambda c: c["name"])
def test_rpb_against_reference_outputs(case):
    """Relative position bias: the oracle against the reference's compat.v014 operators."""
    a = G.arrays(case["name"])
    kw = G.kw(case)
    logits = oracle.na_qk_rpb(a["q"], a["k"], a["rpb"], **kw)
    assert np.abs(logits - a["logits"]).max() < 1e-10
    dq, dk, drpb = oracle.na_qk_rpb_backward(a["q"], a["k"], a["rpb"], a["glog"], **kw)
    for name, got in (("dq", dq), ("dk", dk), ("drpb", drpb)):
        assert np.abs(got - a[name]).max() < 1e-10, name
