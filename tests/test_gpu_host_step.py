"""HostStep (host tensors in, host gradients out, batch slices over three streams) returns
bit-for-bit what the autograd call on device tensors returns."""
import pytest
import torch

from natten_mps_b200 import functional as F
from natten_mps_b200.host_step import HostStep

pytestmark = pytest.mark.gpu


def _host(seed, shapes, dtype):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [torch.randn(s, generator=g).to(dtype).pin_memory() for s in shapes]


@pytest.mark.parametrize("slices", [1, 3, 8])
def test_host_step_2d_bf16_matches_autograd(slices):
    shp = (5, 32, 32, 4, 64)
    q, k, v, go = _host(11, [shp] * 4, torch.bfloat16)
    step = HostStep(2, 7, slices=slices, want_out=True)
    for _ in range(2):                           # second call reuses the staging buffers
        out_h, dq_h, dk_h, dv_h = step(q, k, v, go)
        step.synchronize()
    qd, kd, vd = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    out = F.na2d(qd, kd, vd, 7)
    out.backward(go.cuda())
    for got, want in ((out_h, out), (dq_h, qd.grad), (dk_h, kd.grad), (dv_h, vd.grad)):
        assert torch.equal(got, want.cpu())


def test_host_step_1d_fp32_gqa_causal_stride():
    q, go_full = _host(12, [(3, 96, 4, 32), (3, 48, 4, 32)], torch.float32)
    k, v = _host(13, [(3, 96, 2, 32)] * 2, torch.float32)
    step = HostStep(1, 9, stride=2, is_causal=True, slices=2)
    none_out, dq_h, dk_h, dv_h = step(q, k, v, go_full)
    step.wait()
    torch.cuda.current_stream().synchronize()
    assert none_out is None
    qd, kd, vd = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    F.na1d(qd, kd, vd, 9, stride=2, is_causal=True).backward(go_full.cuda())
    for got, want in ((dq_h, qd.grad), (dk_h, kd.grad), (dv_h, vd.grad)):
        assert torch.equal(got, want.cpu())


def test_host_step_rejects_bad_input():
    step = HostStep(2, 7)
    q, k, v, go = _host(14, [(2, 16, 16, 2, 32)] * 4, torch.float16)
    with pytest.raises(ValueError):
        step(q.cuda(), k, v, go)
    with pytest.raises(ValueError):
        step(q, k, v, go[:, :8])
    with pytest.raises(ValueError):
        HostStep(2, 7)(*_host(15, [(1, 4, 4, 1, 32)] * 4, torch.float16))     # kernel > extent
