"""The five benchmark configurations at full size against the CPU oracle, with the contract's tolerances:
1e-5 relative in float32, 2e-2 absolute for bf16/fp16 outputs and gradients
against a float32 reference on the same rounded inputs."""
import numpy as np
import pytest
import torch

import oracle
from natten_mps_b200 import functional as F
from tests._gpu_util import check

pytestmark = pytest.mark.gpu


def _inputs(seed, shapes, dtype):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [torch.randn(s, generator=g).to(dtype) for s in shapes]


def _run(fn, dtype, q, k, v, go, okw, **kw):
    qd, kd, vd = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    out = fn(qd, kd, vd, **kw)
    out.backward(go.cuda())
    f = lambda t: t.float().numpy()
    ref_out, ref_lse = oracle.na_forward(f(q), f(k), f(v), dtype=np.float32, **okw)
    dq, dk, dv, _, _ = oracle.na_backward(f(q), f(k), f(v), ref_out, ref_lse, f(go), dtype=np.float32, **okw)
    for name, got, want in (("out", out, ref_out), ("dq", qd.grad, dq), ("dk", kd.grad, dk), ("dv", vd.grad, dv)):
        check(name, got, want, dtype)


def test_config1_na1d_fp32():
    q, k, v, go = _inputs(0, [(2, 128, 4, 32)] * 4, torch.float32)
    qd, kd, vd = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    out = F.na1d(qd, kd, vd, 7)
    out.backward(go.cuda())
    f = lambda t: t.double().numpy()
    ref_out, ref_lse = oracle.na_forward(f(q), f(k), f(v), kernel_size=7)
    dq, dk, dv, _, _ = oracle.na_backward(f(q), f(k), f(v), ref_out, ref_lse, f(go), kernel_size=7)
    for name, got, want in (("out", out, ref_out), ("dq", qd.grad, dq), ("dk", kd.grad, dk), ("dv", vd.grad, dv)):
        check(name, got, want, torch.float32)


def test_config2_na2d_bf16_7x7():
    s = (8, 64, 64, 8, 64)
    q, k, v, go = _inputs(0, [s] * 4, torch.bfloat16)
    _run(F.na2d, torch.bfloat16, q, k, v, go, dict(kernel_size=7), kernel_size=7)


def test_config3_na2d_bf16_13x13_dilated_and_strided_forward():
    s = (4, 128, 128, 8, 64)
    q, k, v, go = _inputs(0, [s] * 4, torch.bfloat16)
    _run(F.na2d, torch.bfloat16, q, k, v, go, dict(kernel_size=13, dilation=2), kernel_size=13, dilation=2)
    out = F.na2d(q.cuda(), k.cuda(), v.cuda(), 13, stride=2, dilation=2)
    f = lambda t: t.float().numpy()
    ref, _ = oracle.na_forward(f(q), f(k), f(v), kernel_size=13, stride=2, dilation=2, dtype=np.float32)
    assert out.shape == (4, 64, 64, 8, 64)
    check("strided out", out, ref, torch.bfloat16)


def test_config4_na3d_bf16_causal_depth():
    s = (2, 16, 32, 32, 8, 64)
    q, k, v, go = _inputs(0, [s] * 4, torch.bfloat16)
    kw = dict(kernel_size=(3, 7, 7), is_causal=(True, False, False))
    _run(F.na3d, torch.bfloat16, q, k, v, go, kw, **kw)


def test_config5_na1d_fp16_gqa_varlen_extra_tokens():
    B = 8
    g = torch.Generator(device="cpu").manual_seed(0)
    L, Hq, Hkv, D, K, Ne = 16384, 16, 4, 128, 255, 16
    q = torch.randn((B, L, Hq, D), generator=g).half()
    k = torch.randn((B, L, Hkv, D), generator=g).half()
    v = torch.randn((B, L, Hkv, D), generator=g).half()
    go = torch.randn((B, L, Hq, D), generator=g).half()
    ek = torch.randn((B, Ne, Hkv, D), generator=g).half()
    ev = torch.randn((B, Ne, Hkv, D), generator=g).half()
    lens = torch.randint(4096, 16385, (B,), generator=g, dtype=torch.int32)
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, ek, ev)]
    out = F.na1d_varlen(leaves[0], leaves[1], leaves[2], lens.cuda(), K,
                        additional_keys=leaves[3], additional_values=leaves[4])
    out.backward(go.cuda())
    f = lambda t: t.float().numpy()
    okw = dict(kernel_size=K, additional_keys=f(ek), additional_values=f(ev),
               extents=lens.numpy().reshape(B, 1), dtype=np.float32)
    ref_out, ref_lse = oracle.na_forward(f(q), f(k), f(v), **okw)
    grads = oracle.na_backward(f(q), f(k), f(v), ref_out, ref_lse, f(go), **okw)
    check("out", out, ref_out, torch.float16)
    for name, t, want in zip(("dq", "dk", "dv", "dek", "dev"), leaves, grads):
        if name in ("dek", "dev"):
            # sums over up to 16384*4 queries: compare relative to the tensor's scale
            err = np.abs(t.grad.float().cpu().numpy() - want).max() / max(1.0, np.abs(want).max())
            assert err <= 2e-2, (name, err)
        else:
            check(name, t.grad, want, torch.float16)
    for b in range(B):
        assert float(out[b, int(lens[b]):].abs().sum()) == 0.0
        assert float(leaves[0].grad[b, int(lens[b]):].abs().sum()) == 0.0
