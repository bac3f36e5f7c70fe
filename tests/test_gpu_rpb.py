"""Relative position bias of the split QK operator on the GPU: against the fixtures produced by the
reference's ``compat.v014`` operators (``natten1dqkrpb`` / ``natten2dqkrpb``) and against the oracle,
through the heads-last functions and through the heads-first compat wrappers."""
import numpy as np
import pytest
import torch

import oracle
from natten_mps_b200 import _cabi, functional as F
from natten_mps_b200.compat import v014
from tests import _golden as G
from tests._gpu_util import TOL, dev, rounded

pytestmark = pytest.mark.gpu
FN = {1: F.na1d_qk_rpb, 2: F.na2d_qk_rpb, 3: F.na3d_qk_rpb}


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.bfloat16, torch.float16],
                         ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("case", G.rpb_cases(), ids=lambda c: c["name"])
def test_rpb_against_golden_and_oracle(case, dtype):
    a = G.arrays(case["name"])
    kw = G.kw(case)
    rank = case["rank"]
    q, k, rpb = dev(a["q"], dtype, True), dev(a["k"], dtype, True), dev(a["rpb"], dtype, True)
    logits = FN[rank](q, k, rpb, **kw)
    dq, dk, drpb = torch.autograd.grad((logits.double() * dev(a["glog"], torch.float64)).sum(), [q, k, rpb])
    r = lambda x: rounded(x, dtype)
    want = oracle.na_qk_rpb(r(a["q"]), r(a["k"]), r(a["rpb"]), **kw)
    wdq, wdk, wdrpb = oracle.na_qk_rpb_backward(r(a["q"]), r(a["k"]), r(a["rpb"]), a["glog"], **kw)
    for name, got, ref in (("logits", logits, want), ("dq", dq, wdq), ("dk", dk, wdk), ("drpb", drpb, wdrpb)):
        g = got.detach().double().cpu().numpy()
        err = np.abs(g - ref).max()
        bound = TOL[dtype] * max(1.0, np.abs(ref).max())       # raw dot products / sums: relative to the tensor
        assert err <= bound, (name, err, bound)
    if dtype == torch.float64:                                  # the reference's own numbers
        for name, got in (("logits", logits), ("dq", dq), ("dk", dk), ("drpb", drpb)):
            assert np.abs(got.detach().cpu().numpy() - a[name]).max() < 1e-10, name


TC_CASES = [
    # rank, spatial, kernel, dilation
    (1, (120,), (9,), (2,)),
    (2, (24, 20), (7, 5), (1, 1)),
    (2, (30, 28), (5, 5), (2, 2)),
    (3, (4, 10, 12), (3, 5, 5), (1, 1, 1)),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", TC_CASES, ids=lambda c: "x".join(map(str, c[1])) + f"_k{c[2][-1]}_d{c[3][-1]}")
def test_rpb_inside_the_tensor_core_kernel(case, dtype):
    """Head dim 64 in 16-bit: the bias is added while the tensor-core kernel writes its logits tile out
    (no second pass); compared with the oracle on the rounded inputs and with the two-pass SIMT path."""
    rank, spatial, K, dil = case
    g = torch.Generator().manual_seed(41)
    B, H, D = 2, 2, 64
    q = torch.randn((B, *spatial, H, D), generator=g).to(dtype).cuda()
    k = torch.randn((B, *spatial, H, D), generator=g).to(dtype).cuda()
    rpb = torch.randn((H, *[2 * kk - 1 for kk in K]), generator=g).to(dtype).cuda()
    got = FN[rank](q, k, rpb, K, dil)
    assert _cabi.last_path() == "tcgen05"
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    f = lambda t: t.double().cpu().numpy()
    want = oracle.na_qk_rpb(f(q), f(k), f(rpb), kernel_size=K, dilation=dil)
    g64 = f(got)
    assert np.array_equal(np.isinf(g64), np.isinf(want))
    fin = np.isfinite(want)
    err = np.abs(g64[fin] - want[fin]).max()
    bound = TOL[dtype] * max(1.0, np.abs(want[fin]).max())
    assert err <= bound, (err, bound)
    try:
        _cabi.set_force("simt")
        two_pass = FN[rank](q, k, rpb, K, dil)
        assert _cabi.last_path() == "simt"
    finally:
        _cabi.set_force(None)
    d = (got.float() - two_pass.float())[torch.isfinite(two_pass)].abs().max().item()
    assert d <= bound, d


def test_rpb_rejects_even_kernels():
    q = torch.randn(1, 12, 2, 16, device="cuda")
    with pytest.raises(ValueError, match="odd kernel sizes"):
        F.na1d_qk_rpb(q, q, torch.randn(2, 7, device="cuda"), 4)


def test_compat_wrappers_are_heads_first():
    torch.manual_seed(0)
    B, H, L, D, K = 2, 3, 21, 16, 5
    q, k = torch.randn(B, H, L, D, device="cuda"), torch.randn(B, H, L, D, device="cuda")
    rpb = torch.randn(H, 2 * K - 1, device="cuda")
    got = v014.natten1dqkrpb(q, k, rpb, K, 1)
    assert got.shape == (B, H, L, K)
    ref = F.na1d_qk_rpb(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), rpb, K, 1).permute(0, 2, 1, 3)
    assert torch.equal(got, ref)
    attn = torch.softmax(got, -1)
    v = torch.randn(B, H, L, D, device="cuda")
    out = v014.natten1dav(attn, v, K, 1)
    assert out.shape == (B, H, L, D)
    q2, k2 = torch.randn(1, 2, 9, 8, 16, device="cuda"), torch.randn(1, 2, 9, 8, 16, device="cuda")
    rpb2 = torch.randn(2, 5, 5, device="cuda")
    l2 = v014.natten2dqkrpb(q2, k2, rpb2, 3, 1)
    assert l2.shape == (1, 2, 9, 8, 9)
    o2 = v014.natten2dav(torch.softmax(l2, -1), torch.randn(1, 2, 9, 8, 16, device="cuda"), 3, 1)
    assert o2.shape == (1, 2, 9, 8, 16)
    with pytest.raises(ValueError, match="rpb must have shape"):
        v014.natten1dqkrpb(q, k, rpb[:, :-1], K, 1)


def test_rpb_gradient_is_bit_reproducible_and_3d_runs():
    torch.manual_seed(1)
    q = torch.randn(2, 4, 6, 5, 2, 16, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn_like(q).requires_grad_(True)
    rpb = torch.randn(2, 5, 5, 5, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    grads = []
    for _ in range(2):
        out = F.na3d_qk_rpb(q, k, rpb, 3)
        grads.append(torch.autograd.grad(out.float().square().sum(), [q, k, rpb]))
    for a, b in zip(*grads):
        assert torch.equal(a, b)
    f = lambda t: t.detach().float().cpu().numpy()
    want = oracle.na_qk_rpb(f(q), f(k), f(rpb), 3, dtype=np.float32)
    assert np.abs(f(out) - want).max() <= 2e-2 * max(1.0, np.abs(want).max())
