"""`torch.library` conformance of the custom ops: schema, fake-tensor (Meta) implementations,
autograd registration, AOT dispatch, and one `torch.compile(fullgraph=True)` round trip.
The reference registers the same kind of ops (`src/natten_mps/_torch_ops.py:24-763`) but has
no test that exercises them through `torch.ops` or the compiler."""
import pytest
import torch

import natten_mps_b200  # noqa: F401  (registers torch.ops.natten_b200)
from natten_mps_b200 import functional as F

pytestmark = pytest.mark.gpu

CHECKS = ("test_schema", "test_faketensor", "test_autograd_registration", "test_aot_dispatch_dynamic")


def _t(shape, dtype=torch.float32, grad=True, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(shape, generator=g).to(dtype).cuda().requires_grad_(grad)


def test_opcheck_fused_2d():
    q, k, v = _t((1, 10, 9, 2, 16), seed=1), _t((1, 10, 9, 1, 16), seed=2), _t((1, 10, 9, 1, 16), seed=3)
    args = (q, k, v, None, None, None, [5, 3], [1, 1], [1, 2], [False, True], 0.25)
    torch.library.opcheck(torch.ops.natten_b200.na_fused.default, args, test_utils=CHECKS)


def test_opcheck_fused_1d_extras_extents():
    q, k, v = _t((2, 24, 2, 8), seed=4), _t((2, 24, 2, 8), seed=5), _t((2, 24, 2, 8), seed=6)
    ek, ev = _t((2, 3, 2, 8), seed=7), _t((2, 3, 2, 8), seed=8)
    ext = torch.tensor([[24], [17]], dtype=torch.int32).cuda()
    args = (q, k, v, ek, ev, ext, [7], [1], [1], [False], 0.3)
    torch.library.opcheck(torch.ops.natten_b200.na_fused.default, args, test_utils=CHECKS)


def test_opcheck_split_ops():
    q, k = _t((1, 12, 2, 8), seed=9), _t((1, 12, 2, 8), seed=10)
    torch.library.opcheck(torch.ops.natten_b200.na_qk.default, (q, k, [5], [1], [1], [False], None),
                          test_utils=CHECKS)
    attn = torch.softmax(_t((1, 12, 2, 5), grad=False, seed=11), dim=-1).requires_grad_(True)
    v = _t((1, 12, 2, 8), seed=12)
    torch.library.opcheck(torch.ops.natten_b200.na_av.default, (attn, v, [5], [1], [1], [False]),
                          test_utils=CHECKS)


def test_torch_compile_matches_eager():
    q, k, v = [_t((2, 16, 16, 2, 64), torch.bfloat16, seed=s) for s in (13, 14, 15)]
    go = _t((2, 16, 16, 2, 64), torch.bfloat16, grad=False, seed=16)

    def step(q, k, v):
        return (F.na2d(q, k, v, kernel_size=5) * 2.0).float()

    eager = step(q, k, v)
    eager.backward(go.float())
    want = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    compiled = torch.compile(step, fullgraph=True)
    got = compiled(q, k, v)
    got.backward(go.float())
    assert torch.equal(got, eager)
    for a, b in zip((q.grad, k.grad, v.grad), want):
        assert torch.equal(a, b)
