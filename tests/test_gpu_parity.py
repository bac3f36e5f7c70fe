"""GPU parity: the CUDA path (through the public API and the C ABI) against the
golden fixtures produced by the reference and against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from natten_mps_b200 import _cabi, functional as F
from tests import _golden as G
from natten_mps_b200.utils import normalize_tuple_param as _ntp
from tests._gpu_util import AV, FUSED, QK, check, compare_fused, dev, rounded, run_fused

pytestmark = pytest.mark.gpu

DTYPES = [torch.float64, torch.float32, torch.bfloat16, torch.float16]
PATHS = ["simt", "auto"]


@pytest.fixture(autouse=True)
def _reset_force():
    yield
    _cabi.set_force(None)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("case", G.fused_cases(), ids=lambda c: c["name"])
def test_fused_against_golden_and_oracle(case, dtype, path):
    _cabi.set_force(path)
    a = G.arrays(case["name"])
    kw = G.kw(case)
    got, want = run_fused(case["rank"], dtype, a["q"], a["k"], a["v"], a["gout"], kw,
                          ek=a.get("ek"), ev=a.get("ev"), glse=a.get("glse"))
    compare_fused(got, want, dtype)
    if dtype == torch.float64:
        # the reference's own numbers (float32 merge when extra tokens are present)
        tol_scale = 2e4 if case["n_extra"] else 1.0
        for name in ("out", "dq", "dk", "dv", "dek", "dev", "lse"):
            if name in a and got.get(name) is not None:
                g = got[name].detach().double().cpu().numpy()
                assert np.abs(g - a[name]).max() <= 1e-10 * tol_scale * max(1.0, np.abs(a[name]).max()), name


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("case", G.split_cases(), ids=lambda c: c["name"])
def test_split_ops_against_golden(case, dtype):
    a = G.arrays(case["name"])
    kw = G.kw(case)
    rank = case["rank"]
    q, k, v = dev(a["q"], dtype, True), dev(a["k"], dtype, True), dev(a["v"], dtype, True)
    attn = dev(a["attn"], dtype, True)
    logits = QK[rank](q, k, **kw)
    r = lambda x: rounded(x, dtype)
    want_logits = oracle.na_qk(r(a["q"]), r(a["k"]), **kw)
    check("logits", logits, want_logits, dtype, scale_rel=True)
    glog = dev(a["glog"], dtype)
    finite = torch.isfinite(logits)
    dq, dk = torch.autograd.grad((torch.where(finite, logits, 0.0) * glog).sum(), [q, k])
    wdq, wdk = oracle.na_qk_backward(r(a["q"]), r(a["k"]), r(a["glog"]), **kw)
    check("dq", dq, wdq, dtype, scale_rel=True)
    check("dk", dk, wdk, dtype, scale_rel=True)
    kw.pop("scale", None)
    out = AV[rank](attn, v, **kw)
    check("av_out", out, oracle.na_av(r(a["attn"]), r(a["v"]), **kw), dtype, scale_rel=True)
    dattn, dv = torch.autograd.grad((out * dev(a["gout"], dtype)).sum(), [attn, v])
    wda, wdv = oracle.na_av_backward(r(a["attn"]), r(a["v"]), r(a["gout"]), **kw)
    check("dattn", dattn, wda, dtype, scale_rel=True)
    check("dv", dv, wdv, dtype, scale_rel=True)
    if dtype == torch.float64:
        assert np.abs(logits.detach().cpu().numpy()[np.isfinite(a["logits"])]
                      - a["logits"][np.isfinite(a["logits"])]).max() < 1e-10
        assert np.abs(dk.detach().cpu().numpy() - a["dk"]).max() < 1e-10
        assert np.abs(dv.detach().cpu().numpy() - a["dv"]).max() < 1e-10


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("case", G.varlen_cases(), ids=lambda c: c["name"])
def test_varlen_against_golden(case, dtype, path):
    _cabi.set_force(path)
    a = G.arrays(case["name"])
    got, want = run_fused(case["rank"], dtype, a["q"], a["k"], a["v"], a["gout"], G.kw(case),
                          sizes=case["sizes"])
    got["lse"] = None
    compare_fused(got, want, dtype)
    if dtype == torch.float64:
        for name in ("out", "dq", "dk", "dv"):
            assert np.abs(got[name].detach().cpu().numpy() - a[name]).max() < 1e-10, name
    # rows past each sample's extent are exactly zero, forward and backward
    sizes = case["sizes"]
    for b, ext in enumerate(sizes):
        mask = np.ones(a["q"].shape[1:1 + case["rank"]], dtype=bool)
        mask[tuple(slice(0, e) for e in ext)] = False
        for name in ("out", "dq", "dk", "dv"):
            assert float(got[name][b].detach().abs().double().cpu().numpy()[mask].sum()) == 0.0


RANDOM_CASES = [
    # rank, spatial, B, Hq, Hkv, D, Dv, kwargs, n_extra, sizes
    (1, (70,), 2, 4, 2, 64, 64, dict(kernel_size=9), 0, None),
    (1, (61,), 2, 4, 1, 17, 17, dict(kernel_size=7, dilation=2), 3, None),          # odd D: scalar loads
    (1, (96,), 3, 8, 2, 128, 128, dict(kernel_size=31), 5, [[96], [40], [77]]),     # varlen+GQA+extras
    (2, (20, 18), 2, 4, 4, 64, 64, dict(kernel_size=7), 0, None),
    (2, (17, 21), 1, 2, 2, 32, 32, dict(kernel_size=(5, 3), dilation=(2, 3), stride=(2, 1),
                                        is_causal=(False, True)), 0, None),
    (2, (16, 16), 2, 4, 2, 64, 64, dict(kernel_size=5), 2, [[16, 16], [9, 12]]),
    (3, (6, 10, 9), 1, 4, 2, 64, 64, dict(kernel_size=(3, 5, 5), is_causal=(True, False, False)), 0, None),
    (3, (5, 8, 8), 1, 2, 2, 200, 200, dict(kernel_size=3, dilation=(1, 2, 2)), 0, None),
    (2, (12, 12), 1, 2, 2, 64, 64, dict(kernel_size=(4, 6)), 0, None),              # even kernels
    (1, (150,), 2, 4, 2, 64, 64, dict(kernel_size=12), 0, None),
    (3, (5, 12, 14), 1, 2, 2, 64, 64, dict(kernel_size=(2, 4, 6), is_causal=(True, False, False)), 0, None),
    (2, (22, 26), 3, 4, 2, 64, 64, dict(kernel_size=5, dilation=2), 0, [[22, 26], [10, 15], [13, 10]]),   # varlen + dilation
    (1, (90,), 2, 2, 2, 128, 128, dict(kernel_size=7, dilation=3), 0, [[90], [21]]),
    (2, (28, 28), 2, 4, 2, 32, 32, dict(kernel_size=7), 2, None),                   # head dim 32: padded tensor-core path
    (1, (200,), 2, 4, 4, 96, 96, dict(kernel_size=15, dilation=2), 0, None),        # head dim 96
]


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16],
                         ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("case", RANDOM_CASES, ids=lambda c: f"r{c[0]}_{'x'.join(map(str, c[1]))}_d{c[5]}")
def test_fused_against_oracle_random(case, dtype, path):
    _cabi.set_force(path)
    rank, spatial, B, Hq, Hkv, D, Dv, kw, n_extra, sizes = case
    rng = np.random.default_rng(hash((rank, spatial, D)) % (2 ** 31))
    q = rng.standard_normal((B, *spatial, Hq, D))
    k = rng.standard_normal((B, *spatial, Hkv, D))
    v = rng.standard_normal((B, *spatial, Hkv, Dv))
    gout = rng.standard_normal((B, *[(n + s - 1) // s for n, s in
                                     zip(spatial, _ntp(kw.get("stride", 1), rank, "stride"))],
                                Hq, Dv))
    ek = ev = None
    if n_extra:
        ek = rng.standard_normal((B, n_extra, Hkv, D))
        ev = rng.standard_normal((B, n_extra, Hkv, Dv))
    glse = None if sizes is not None else rng.standard_normal(gout.shape[:-1])
    got, want = run_fused(rank, dtype, q, k, v, gout, kw, ek=ek, ev=ev, glse=glse, sizes=sizes)
    if sizes is not None:
        got["lse"] = None
    compare_fused(got, want, dtype)


def test_strided_views_from_a_fused_projection_need_no_copy():
    torch.manual_seed(0)
    B, H, W, heads, D = 2, 10, 12, 4, 32
    qkv = torch.randn(B, H, W, 3, heads, D, device="cuda")
    q, k, v = qkv.unbind(dim=3)
    assert _cabi.token_strides(q, 2) == (H * W * 3 * heads * D, 3 * heads * D, D)
    out = F.na2d(q, k, v, 5)
    ref = F.na2d(q.contiguous(), k.contiguous(), v.contiguous(), 5)
    assert torch.equal(out, ref)


def test_backward_is_bit_reproducible():
    torch.manual_seed(1)
    q, k, v, go = [torch.randn(2, 24, 24, 4, 64, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    grads = []
    for _ in range(2):
        qq, kk, vv = [t.clone().requires_grad_(True) for t in (q, k, v)]
        F.na2d(qq, kk, vv, 7).backward(go)
        grads.append((qq.grad, kk.grad, vv.grad))
    for a, b in zip(*grads):
        assert torch.equal(a, b)


def test_global_attention_when_kernel_covers_input():
    torch.manual_seed(2)
    q, k, v = [torch.randn(2, 9, 4, 16, device="cuda") for _ in range(3)]
    out = F.na1d(q, k, v, 9)
    want = torch.softmax(torch.einsum("blhd,bmhd->bhlm", q, k) * 16 ** -0.5, -1)
    want = torch.einsum("bhlm,bmhd->blhd", want, v)
    assert torch.allclose(out, want, atol=1e-5)


def test_causal_first_position_sees_only_itself():
    torch.manual_seed(3)
    q, k, v = [torch.randn(1, 12, 2, 8, device="cuda") for _ in range(3)]
    out = F.na1d(q, k, v, 5, is_causal=True)
    assert torch.allclose(out[:, 0], v[:, 0], atol=1e-6)


def test_module_forward_backward_and_gqa():
    import natten_mps_b200 as nb
    torch.manual_seed(4)
    for m, x in ((nb.NeighborhoodAttention2D(64, 4, 5).cuda(), torch.randn(2, 12, 12, 64, device="cuda")),
                 (nb.NeighborhoodAttention1D(64, 4, 5, num_kv_heads=2).cuda(), torch.randn(2, 20, 64, device="cuda")),
                 (nb.NeighborhoodAttention3D(32, 2, 3, attn_drop=0.1).cuda(), torch.randn(1, 4, 6, 6, 32, device="cuda"))):
        x.requires_grad_(True)
        y = m(x)
        assert y.shape == x.shape
        y.sum().backward()
        assert x.grad is not None and torch.isfinite(x.grad).all()
        assert all(p.grad is not None for p in m.parameters())


def test_gradcheck_float64():
    torch.manual_seed(5)
    q, k, v = [torch.randn(1, 7, 2, 4, device="cuda", dtype=torch.float64, requires_grad=True) for _ in range(3)]
    assert torch.autograd.gradcheck(lambda a, b, c: F.na1d(a, b, c, 3, dilation=2), (q, k, v), atol=1e-6)
    q2, k2, v2 = [torch.randn(1, 4, 5, 2, 4, device="cuda", dtype=torch.float64, requires_grad=True) for _ in range(3)]
    assert torch.autograd.gradcheck(
        lambda a, b, c: F.na2d(a, b, c, 3, is_causal=(True, False), return_lse=True), (q2, k2, v2), atol=1e-6)
    assert torch.autograd.gradcheck(lambda a, b: F.na2d_qk(a, b, 3, scale=0.7), (q2, k2), atol=1e-6)
    attn = torch.randn(1, 4, 5, 2, 9, device="cuda", dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a, b: F.na2d_av(a, b, 3), (attn, v2), atol=1e-6)
