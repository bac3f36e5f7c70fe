"""The no-allocation backward entry point (``natten_fused_bwd_static``).

It exists for hosts that may not allocate device memory when the backward runs
(fully handed-out memory pools, plugins that only receive their buffers): the
scratch the backward needs lives in a fixed array inside the library.  Called here
straight through the C ABI, twice in a row, and compared with the regular entry
point, which receives a caller-allocated workspace.  The file name keeps it last in
collection order; it does not depend on anything the other tests leave behind.
"""
import ctypes

import pytest
import torch

from natten_mps_b200 import _backend, _cabi

pytestmark = pytest.mark.gpu


def _problem(seed, dtype, spatial, heads, kv_heads, dim):
    g = torch.Generator(device="cpu").manual_seed(seed)
    mk = lambda h: torch.randn((2, *spatial, h, dim), generator=g).to(dtype).cuda()
    return mk(heads), mk(kv_heads), mk(kv_heads), mk(heads)


def _static_backward(q, k, v, out, lse, dout, ks, st, dil, causal, scale):
    rank = q.ndim - 3
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    p = _cabi.make_params(rank, q.dtype, q.shape[0], q.shape[-2], k.shape[-2], q.shape[-1], v.shape[-1],
                          q.shape[1:1 + rank], ks, st, dil, causal, scale, 0,
                          _cabi.token_strides(q, rank), _cabi.token_strides(k, rank),
                          _cabi.token_strides(v, rank))
    rc = _cabi.lib().natten_fused_bwd_static(
        p, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), None, None, _cabi.ptr(out), _cabi.ptr(lse),
        _cabi.ptr(dout), None, _cabi.ptr(dq), _cabi.ptr(dk), _cabi.ptr(dv), None, None,
        _cabi.stream_of(q))
    return rc, dq, dk, dv


@pytest.mark.parametrize("dtype,spatial,dim", [(torch.bfloat16, (24, 20), 64), (torch.float32, (50,), 32)],
                         ids=["bf16_2d_tensor_cores", "f32_1d_simt"])
def test_static_scratch_backward_matches_regular_entry_point(dtype, spatial, dim):
    rank = len(spatial)
    ks, st, dil, causal, scale = (5,) * rank, (1,) * rank, (1,) * rank, (False,) * rank, dim ** -0.5
    for call in range(2):                                    # two calls in a row share the scratch
        q, k, v, dout = _problem(100 + call, dtype, spatial, 4, 2, dim)
        out, lse = _backend.fused_forward(q, k, v, ks, st, dil, causal, scale)
        want = _backend.fused_backward(q, k, v, out, lse, dout, ks, st, dil, causal, scale)
        rc, dq, dk, dv = _static_backward(q, k, v, out, lse, dout, ks, st, dil, causal, scale)
        assert rc == 0, _cabi.lib().natten_strerror(rc)
        torch.cuda.synchronize()
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5      # same bounds as the other parity tests
        for name, a, b in zip(("dq", "dk", "dv"), (dq, dk, dv), want[:3]):
            err = (a.float() - b.float()).abs().max().item()
            assert err <= tol * max(1.0, b.float().abs().max().item()), (name, call, err)


def test_static_scratch_rejects_oversized_problems():
    limit = _cabi.lib().natten_static_scratch_bytes()
    assert limit == 4 << 20
    rows = limit // 4 + 1024                                 # one float of scratch per (batch, query, head)
    p = _cabi.make_params(1, torch.float32, 1, 1, 1, 8, 8, (rows,), (3,), (1,), (1,), (False,), 0.5)
    rc = _cabi.lib().natten_fused_bwd_static(p, *([None] * 15))
    assert rc == -5
    assert b"built-in scratch" in _cabi.lib().natten_strerror(rc)


def test_static_scratch_limit_follows_the_workspace_size():
    """The limit is the workspace size, not a row count: double precision needs 8 bytes per row and
    additional tokens add their partial sums."""
    L = _cabi.lib()
    limit = L.natten_static_scratch_bytes()
    rows_f64 = limit // 8
    fits = _cabi.make_params(1, torch.float64, 1, 1, 1, 8, 8, (rows_f64,), (3,), (1,), (1,), (False,), 0.5)
    over = _cabi.make_params(1, torch.float64, 1, 1, 1, 8, 8, (rows_f64 + 64,), (3,), (1,), (1,), (False,), 0.5)
    assert L.natten_workspace_bytes(fits, _cabi.OP_FUSED_BWD) <= limit
    assert L.natten_workspace_bytes(over, _cabi.OP_FUSED_BWD) > limit
    assert L.natten_fused_bwd_static(over, *([None] * 15)) == -5
    assert L.natten_fused_bwd_static(fits, *([None] * 15)) == -1      # passes the size check, then null pointers
    extra = _cabi.make_params(1, torch.float32, 1, 4, 4, 64, 64, (limit // 16,), (3,), (1,), (1,), (False,), 0.5,
                              n_extra=8)
    need = L.natten_workspace_bytes(extra, _cabi.OP_FUSED_BWD)
    assert need > limit // 16 * 4 * 4                                  # more than the delta rows alone
    assert (L.natten_fused_bwd_static(extra, *([None] * 15)) == -5) == (need > limit)


def test_static_scratch_backward_in_double_precision_with_additional_tokens():
    dtype, spatial, dim, ne = torch.float64, (40,), 16, 3
    ks, st, dil, causal, scale = (5,), (1,), (1,), (False,), dim ** -0.5
    for call in range(2):
        q, k, v, dout = _problem(200 + call, dtype, spatial, 4, 2, dim)
        g = torch.Generator(device="cpu").manual_seed(300 + call)
        ek = torch.randn((2, ne, 2, dim), generator=g).to(dtype).cuda()
        ev = torch.randn((2, ne, 2, dim), generator=g).to(dtype).cuda()
        out, lse = _backend.fused_forward(q, k, v, ks, st, dil, causal, scale, extra_k=ek, extra_v=ev)
        want = _backend.fused_backward(q, k, v, out, lse, dout, ks, st, dil, causal, scale, extra_k=ek, extra_v=ev)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dek, dev = torch.empty_like(ek), torch.empty_like(ev)
        p = _cabi.make_params(1, dtype, 2, 4, 2, dim, dim, spatial, ks, st, dil, causal, scale, ne,
                              _cabi.token_strides(q, 1), _cabi.token_strides(k, 1), _cabi.token_strides(v, 1))
        rc = _cabi.lib().natten_fused_bwd_static(
            p, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(ek), _cabi.ptr(ev), _cabi.ptr(out), _cabi.ptr(lse),
            _cabi.ptr(dout), None, _cabi.ptr(dq), _cabi.ptr(dk), _cabi.ptr(dv), _cabi.ptr(dek), _cabi.ptr(dev),
            _cabi.stream_of(q))
        assert rc == 0, _cabi.lib().natten_strerror(rc)
        torch.cuda.synchronize()
        for name, a, b in zip(("dq", "dk", "dv", "dek", "dev"), (dq, dk, dv, dek, dev), want):
            err = (a - b).abs().max().item()
            assert err <= 1e-10 * max(1.0, b.abs().max().item()), (name, call, err)
