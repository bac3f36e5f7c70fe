"""Failure reporting of the tensor-core kernels, per-device launcher state, and padding hygiene.

* A barrier wait that runs out must surface as an error and must be recoverable.  The failure is
  made on the host: a test hook lets the fused forward's first barrier expect more bytes than its
  loads deliver and shortens the wait budget to a fraction of a millisecond, so the wait gives up
  (it never hangs), the kernel returns with the device's status word set, the next call raises,
  and after ``clear_status()`` the same call computes correctly again.
* One process using two GPUs in turn (skipped with a single GPU).
* Per-sample extents: whatever sits in the padding rows (NaN here) must not reach the results,
  which the reference guarantees by slicing each sample (``src/natten_mps/_core/pure.py:586-599``).
"""
import numpy as np
import pytest
import torch

import oracle
from natten_mps_b200 import _backend, _cabi, functional as F

pytestmark = pytest.mark.gpu


def _case(seed=0, B=2, H=24, W=40, heads=2, D=64, dtype=torch.bfloat16, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(B, H, W, heads, D, generator=g).to(dtype).to(device) for _ in range(3)]


def _oracle_out(q, k, v, K):
    f = lambda t: t.detach().float().cpu().numpy()
    return oracle.na_forward(f(q), f(k), f(v), kernel_size=K, dtype=np.float32)[0]


def test_wait_that_runs_out_is_reported_and_recoverable():
    q, k, v = _case()
    args = (q, k, v, (7, 7), (1, 1), (1, 1), (False, False), 0.125)
    L = _cabi.lib()
    try:
        L.natten_debug_wait(400_000, 1)           # ~0.2 ms budget; first barrier can never complete
        _cabi.set_force("tc")
        _backend.fused_forward(*args)
        assert _cabi.last_path() == "tcgen05"
        torch.cuda.synchronize()                  # returns: the kernel gave up instead of hanging
        assert _cabi.device_status() == -4        # NATTEN_E_DEVICE
        with pytest.raises(RuntimeError, match="bounded wait"):
            _backend.fused_forward(*args)         # the front end refuses to go on silently
    finally:
        L.natten_debug_wait(0, 0)
        _cabi.set_force(None)
        _cabi.clear_status()
    assert _cabi.device_status() == 0
    out, _ = _backend.fused_forward(*args)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    err = np.abs(out.float().cpu().numpy() - _oracle_out(q, k, v, 7)).max()
    assert err <= 2e-2, err


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_devices_in_one_process():
    for dev in ("cuda:0", "cuda:1", "cuda:0"):
        q, k, v = _case(seed=3, device=dev)
        qq, kk, vv = [t.requires_grad_(True) for t in (q, k, v)]
        out = F.na2d(qq, kk, vv, 7)
        out.sum().backward()
        torch.cuda.synchronize(dev)
        assert _cabi.last_path() == "tcgen05"
        err = np.abs(out.detach().float().cpu().numpy() - _oracle_out(q, k, v, 7)).max()
        assert err <= 2e-2, (dev, err)
        assert torch.isfinite(qq.grad).all() and torch.isfinite(kk.grad).all()


@pytest.mark.parametrize("path", ["simt", "auto"])
@pytest.mark.parametrize("rank,D,dtype", [(1, 128, torch.float16), (2, 64, torch.bfloat16), (1, 32, torch.float32)],
                         ids=["1d_d128_f16", "2d_d64_bf16", "1d_d32_f32"])
def test_padding_rows_never_reach_the_results(rank, D, dtype, path):
    g = torch.Generator().manual_seed(11)
    if rank == 1:
        spatial, K, sizes = (300,), 31, [[300], [77], [200]]
    else:
        spatial, K, sizes = (20, 24), 5, [[20, 24], [9, 13], [16, 7]]
    B, Hq, Hkv = len(sizes), 4, 2
    mk = lambda h: torch.randn(B, *spatial, h, D, generator=g).to(dtype)
    q, k, v, go = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    f = lambda t: t.float().numpy()
    okw = dict(kernel_size=K, extents=np.asarray(sizes), dtype=np.float32)
    ref_out, ref_lse = oracle.na_forward(f(q), f(k), f(v), **okw)
    ref = (ref_out,) + oracle.na_backward(f(q), f(k), f(v), ref_out, ref_lse, f(go), **okw)[:3]
    # poison everything outside each sample's extent
    pad = torch.ones(B, *spatial, dtype=torch.bool)
    for b, ext in enumerate(sizes):
        pad[(b, *[slice(0, e) for e in ext])] = False
    for t in (q, k, v, go):
        t[pad] = float("nan")
    _cabi.set_force(path)
    try:
        leaves = [t.cuda().requires_grad_(True) for t in (q, k, v)]
        st = torch.tensor(sizes, dtype=torch.int32).cuda()
        fn = F.na1d_varlen if rank == 1 else F.na2d_varlen
        out = fn(*leaves, st[:, 0] if rank == 1 else st, K)
        grads = torch.autograd.grad(out, leaves, go.cuda())
    finally:
        _cabi.set_force(None)
    tol = 2e-2 if dtype != torch.float32 else 1e-4
    for name, got, want in zip(("out", "dq", "dk", "dv"), (out, *grads), ref):
        got = got.detach().float().cpu()
        assert torch.isfinite(got).all(), f"{name}: padding leaked into the result"
        assert float(got[pad].abs().sum()) == 0.0, f"{name}: padded rows must be exactly zero"
        err = float((got - torch.as_tensor(want)).abs().max())
        assert err <= tol * max(1.0, float(np.abs(want).max())) if dtype == torch.float32 else err <= tol, (name, err)
