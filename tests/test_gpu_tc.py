"""The tcgen05 kernels against the SIMT kernels (and through them the oracle) on
shapes that exercise tile edges, dilation sub-grids, causal axes, GQA and
per-sample extents.  Each case asserts that the tensor-core path really ran."""
import pytest
import torch

from natten_mps_b200 import _backend, _cabi

pytestmark = pytest.mark.gpu

CASES = [
    # spatial, B, Hq, Hkv, kernel, dilation, causal, extents
    ((64, 64), 2, 2, 2, (7, 7), (1, 1), (False, False), None),
    ((20, 19), 1, 2, 1, (7, 5), (1, 1), (False, False), None),          # ragged tiles, GQA
    ((33, 40), 1, 2, 2, (13, 13), (1, 1), (False, False), None),
    ((30, 28), 1, 2, 2, (5, 5), (2, 2), (False, False), None),          # dilation sub-grids
    ((27, 31), 1, 1, 1, (3, 7), (3, 2), (True, False), None),           # dilation, ragged, causal
    ((24, 24), 2, 2, 2, (5, 7), (1, 1), (True, True), None),
    ((24, 24), 3, 2, 2, (5, 5), (1, 1), (False, False), [[24, 24], [9, 17], [5, 5]]),
    ((300,), 2, 4, 2, (31,), (1,), (False,), None),
    ((700,), 1, 2, 2, (255,), (1,), (False,), None),
    ((500,), 2, 2, 2, (63,), (1,), (True,), [[500], [260]]),
    ((100,), 1, 2, 2, (9,), (2,), (False,), None),
    ((6, 20, 18), 1, 2, 2, (3, 7, 7), (1, 1, 1), (True, False, False), None),
    ((5, 9, 11), 1, 2, 1, (3, 3, 5), (1, 2, 1), (False, False, False), None),
    ((8, 12, 12), 2, 1, 1, (3, 5, 5), (1, 1, 1), (False, False, False), [[8, 12, 12], [4, 7, 9]]),
    # even kernel sizes: the clamped window stops one short of the last key; the last key has no query
    ((40, 36), 1, 2, 2, (4, 6), (1, 1), (False, False), None),
    ((26, 33), 2, 2, 1, (8, 5), (1, 2), (False, False), None),          # even on the undilated axis only
    ((200,), 2, 2, 2, (32,), (1,), (False,), None),
    ((9, 9), 1, 1, 1, (8, 8), (1, 1), (False, False), None),            # L = K + 1
    ((6, 14, 20), 1, 2, 2, (2, 4, 6), (1, 1, 1), (True, False, False), None),
    # per-sample extents together with dilation
    ((30, 28), 3, 2, 2, (5, 5), (2, 2), (False, False), [[30, 28], [11, 17], [10, 10]]),
    ((400,), 3, 2, 1, (15,), (2,), (False,), [[400], [61], [233]]),
    ((8, 14, 12), 2, 1, 1, (3, 3, 5), (2, 1, 2), (False, False, False), [[8, 14, 12], [6, 7, 10]]),
    # head dim 128 (ninth field)
    ((40, 24), 1, 2, 1, (7, 7), (1, 1), (False, False), None, 128),
    ((600,), 2, 4, 1, (255,), (1,), (False,), [[600], [300]], 128),
    ((5, 9, 17), 1, 2, 2, (3, 5, 7), (1, 1, 1), (True, False, False), None, 128),
    ((26, 30), 1, 2, 2, (5, 5), (2, 2), (False, False), None, 128),
    # head dims that run zero-padded on the 64 / 128 kernels (ranks 1 and 2)
    ((28, 28), 2, 4, 2, (7, 7), (1, 1), (False, False), None, 32),
    ((24, 24), 2, 2, 2, (5, 5), (1, 1), (False, False), [[24, 24], [9, 17]], 32),
    ((400,), 2, 4, 2, (63,), (1,), (False,), [[400], [123]], 48),
    ((20, 19), 1, 2, 1, (5, 5), (2, 1), (True, False), None, 96),
    ((300,), 1, 2, 2, (31,), (1,), (False,), None, 8),
]


def _dim(case):
    return case[8] if len(case) > 8 else 64


def _id(c):
    return "x".join(map(str, c[0])) + f"_k{c[4][0]}_d{c[5][0]}_h{_dim(c)}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", CASES, ids=_id)
def test_tc_forward_matches_simt(case, dtype):
    spatial, B, Hq, Hkv, ks, dil, causal, extents = case[:8]
    D = _dim(case)
    rank = len(spatial)
    g = torch.Generator(device="cpu").manual_seed(7)
    q = torch.randn((B, *spatial, Hq, D), generator=g).to(dtype).cuda()
    k = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    v = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    ext = None if extents is None else torch.tensor(extents, dtype=torch.int32).cuda()
    args = (q, k, v, ks, (1,) * rank, dil, causal, D ** -0.5)
    try:
        _cabi.set_force("simt")
        ref_out, ref_lse = _backend.fused_forward(*args, extents=ext)
        _cabi.set_force("tc")
        out, lse = _backend.fused_forward(*args, extents=ext)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    err = (out.float() - ref_out.float()).abs().max().item()
    lerr = (lse - ref_lse).abs().max().item()
    assert err <= 1.6e-2, f"out differs by {err}"
    assert lerr <= 2e-3, f"lse differs by {lerr}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", CASES, ids=_id)
def test_tc_backward_matches_simt(case, dtype):
    spatial, B, Hq, Hkv, ks, dil, causal, extents = case[:8]
    D = _dim(case)
    rank = len(spatial)
    g = torch.Generator(device="cpu").manual_seed(11)
    q = torch.randn((B, *spatial, Hq, D), generator=g).to(dtype).cuda()
    k = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    v = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    go = torch.randn((B, *spatial, Hq, D), generator=g).to(dtype).cuda()
    glse = torch.randn((B, *spatial, Hq), generator=g).cuda()
    ext = None if extents is None else torch.tensor(extents, dtype=torch.int32).cuda()
    geo = (ks, (1,) * rank, dil, causal, D ** -0.5)
    try:
        _cabi.set_force("simt")
        out, lse = _backend.fused_forward(q, k, v, *geo, extents=ext)
        ref = _backend.fused_backward(q, k, v, out, lse, go, *geo, extents=ext, dlse=glse)
        _cabi.set_force("tc")
        got = _backend.fused_backward(q, k, v, out, lse, go, *geo, extents=ext, dlse=glse)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    for name, a, r in zip(("dq", "dk", "dv"), got[:3], ref[:3]):
        err = (a.float() - r.float()).abs().max().item()
        scale = max(1.0, r.float().abs().max().item())
        assert err <= 2e-2 * scale, f"{name} differs by {err} (scale {scale})"


EXTRA_CASES = [
    # spatial, B, Hq, Hkv, D, kernel, n_extra, extents
    ((400,), 2, 4, 1, 128, (63,), 16, [[400], [170]]),
    ((20, 24), 2, 2, 2, 64, (7, 7), 3, None),
    ((300,), 1, 2, 2, 64, (31,), 130, None),          # more than one chunk of additional tokens
    ((4, 10, 12), 1, 2, 1, 64, (3, 5, 5), 20, None),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", EXTRA_CASES, ids=lambda c: "x".join(map(str, c[0])) + f"_e{c[6]}_h{c[4]}")
def test_tc_additional_tokens_match_simt(case, dtype):
    spatial, B, Hq, Hkv, D, ks, n_extra, extents = case
    rank = len(spatial)
    g = torch.Generator(device="cpu").manual_seed(23)
    mk = lambda *shape: torch.randn(shape, generator=g).to(dtype).cuda()
    q, k, v = mk(B, *spatial, Hq, D), mk(B, *spatial, Hkv, D), mk(B, *spatial, Hkv, D)
    ek, ev, go = mk(B, n_extra, Hkv, D), mk(B, n_extra, Hkv, D), mk(B, *spatial, Hq, D)
    ext = None if extents is None else torch.tensor(extents, dtype=torch.int32).cuda()
    geo = (ks, (1,) * rank, (1,) * rank, (False,) * rank, D ** -0.5)
    kw = dict(extra_k=ek, extra_v=ev, extents=ext)
    try:
        _cabi.set_force("simt")
        ref_out, ref_lse = _backend.fused_forward(q, k, v, *geo, **kw)
        ref = _backend.fused_backward(q, k, v, ref_out, ref_lse, go, *geo, **kw)
        _cabi.set_force("tc")
        out, lse = _backend.fused_forward(q, k, v, *geo, **kw)
        assert _cabi.last_path() == "tcgen05"
        got = _backend.fused_backward(q, k, v, ref_out, ref_lse, go, *geo, **kw)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    assert (out.float() - ref_out.float()).abs().max().item() <= 1.6e-2
    assert (lse - ref_lse).abs().max().item() <= 2e-3
    for name, a, r in zip(("dq", "dk", "dv", "dek", "dev"), got, ref):
        err = (a.float() - r.float()).abs().max().item()
        scale = max(1.0, r.float().abs().max().item())
        assert err <= 2e-2 * scale, f"{name} differs by {err} (scale {scale})"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("spatial,ks,slope,axis", [((700,), (255,), 12.0 / 128.0, -1), ((40, 48), (13, 13), 1.0, -1),
                                                   ((40, 48), (13, 13), 4.0, -1), ((48, 40), (7, 7), 12.0, 0)],
                         ids=["1d", "2d", "2d_steep", "2d_k7_rows"])
def test_tc_forward_rescales_when_later_chunks_dominate(spatial, ks, slope, axis, D, dtype):
    """Scores that grow steeply along one key axis (`slope` per key along `axis`): later chunks of a tile
    raise the row maximum by far more than the stored probabilities may exceed their stabiliser by (2^14
    for fp16 and 2^60 for bf16, which the steep cases exceed), so the output accumulated in TMEM has to be
    rescaled.  The 7 x 7 case ramps along the rows, which are the 16-column pieces of its chunks: the
    rescale then happens on the kernel's 16-column fast path."""
    rank = len(spatial)
    B, H = 2, 2
    g = torch.Generator(device="cpu").manual_seed(23)
    axis = axis % rank
    shape = [1] * rank + [1, 1]
    shape[axis] = spatial[axis]
    ramp = (torch.arange(spatial[axis], dtype=torch.float32) * slope).reshape(shape)
    q = torch.randn((B, *spatial, H, D), generator=g) * 0.1 + 1.0
    k = torch.randn((B, *spatial, H, D), generator=g) * 0.1 + ramp.unsqueeze(0) / (D ** 0.5)
    v = torch.randn((B, *spatial, H, D), generator=g)
    q, k, v = [t.to(dtype).cuda() for t in (q, k, v)]
    args = (q, k, v, ks, (1,) * rank, (1,) * rank, (False,) * rank, D ** -0.5)
    try:
        _cabi.set_force("simt")
        ref_out, ref_lse = _backend.fused_forward(*args)
        _cabi.set_force("tc")
        out, lse = _backend.fused_forward(*args)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    # the window's scores really span far more than 2^8
    assert (ref_lse.max() - ref_lse.min()).item() > 20.0
    err = (out.float() - ref_out.float()).abs().max().item()
    lerr = ((lse - ref_lse).abs() / ref_lse.abs().clamp(min=1.0)).max().item()
    assert err <= 2e-2, f"out differs by {err}"
    assert lerr <= 2e-3, f"lse differs by {lerr} (relative)"


STRIDE_CASES = [
    # spatial, B, Hq, Hkv, kernel, dilation, stride, causal, extents, D
    ((64, 64), 1, 2, 2, (13, 13), (2, 2), (2, 2), (False, False), None, 64),     # config 3's strided variant, small
    ((40, 36), 2, 2, 1, (7, 7), (1, 1), (2, 2), (False, False), None, 64),       # stride without dilation, GQA
    ((37, 41), 1, 2, 2, (5, 7), (2, 3), (3, 2), (False, True), None, 64),        # coprime stride / dilation, ragged, causal
    ((48, 40), 1, 1, 1, (5, 5), (2, 2), (4, 4), (False, False), None, 64),       # stride a multiple of the dilation
    ((300,), 2, 4, 2, (31,), (1,), (2,), (False,), [[300], [170]], 64),          # 1-D, per-sample lengths
    ((6, 20, 18), 1, 2, 2, (3, 7, 5), (1, 1, 2), (1, 2, 3), (True, False, False), None, 64),
    ((33, 30), 1, 2, 1, (7, 7), (1, 1), (3, 2), (False, False), None, 128),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", STRIDE_CASES, ids=lambda c: "x".join(map(str, c[0])) + f"_s{c[6][-1]}_d{c[5][-1]}_h{c[9]}")
def test_tc_forward_with_output_stride_matches_simt(case, dtype):
    spatial, B, Hq, Hkv, ks, dil, st, causal, extents, D = case
    g = torch.Generator(device="cpu").manual_seed(29)
    q = torch.randn((B, *spatial, Hq, D), generator=g).to(dtype).cuda()
    k = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    v = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    ext = None if extents is None else torch.tensor(extents, dtype=torch.int32).cuda()
    args = (q, k, v, ks, st, dil, causal, D ** -0.5)
    try:
        _cabi.set_force("simt")
        ref_out, ref_lse = _backend.fused_forward(*args, extents=ext)
        _cabi.set_force("tc")
        out, lse = _backend.fused_forward(*args, extents=ext)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    assert out.shape == ref_out.shape == (B, *[-(-n // s) for n, s in zip(spatial, st)], Hq, D)
    err = (out.float() - ref_out.float()).abs().max().item()
    lerr = (lse - ref_lse).abs().max().item()
    assert err <= 1.6e-2, f"out differs by {err}"
    assert lerr <= 2e-3, f"lse differs by {lerr}"


SPLIT_CASES = [
    # spatial, B, Hq, Hkv, kernel, dilation, stride, causal, D
    ((64, 64), 2, 2, 2, (7, 7), (1, 1), (1, 1), (False, False), 64),
    ((20, 19), 1, 2, 1, (7, 5), (1, 1), (1, 1), (False, False), 64),            # ragged tiles, GQA
    ((33, 40), 1, 2, 2, (13, 13), (2, 2), (1, 1), (False, False), 64),          # 169 slots, dilation
    ((27, 31), 1, 1, 1, (3, 7), (3, 2), (1, 1), (True, False), 64),             # causal axis: masked slots
    ((40, 36), 1, 2, 2, (5, 5), (1, 1), (2, 2), (False, True), 64),             # output stride
    ((300,), 2, 4, 2, (31,), (1,), (1,), (False,), 64),
    ((260,), 1, 2, 2, (63,), (1,), (1,), (True,), 128),
    ((6, 20, 18), 1, 2, 2, (3, 7, 7), (1, 1, 1), (1, 1, 1), (True, False, False), 64),     # 147 slots
    ((5, 9, 11), 1, 2, 1, (3, 3, 5), (1, 2, 1), (1, 1, 1), (False, False, False), 128),
    ((30, 22), 1, 2, 2, (6, 4), (1, 1), (1, 1), (False, False), 64),            # even kernels
    ((120,), 2, 2, 1, (16,), (1,), (1,), (False,), 64),
]


def _split_id(c):
    return "x".join(map(str, c[0])) + f"_k{c[4][-1]}_d{c[5][-1]}_s{c[6][-1]}_h{c[8]}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", SPLIT_CASES, ids=_split_id)
def test_tc_qk_forward_matches_simt(case, dtype):
    spatial, B, Hq, Hkv, ks, dil, st, causal, D = case
    g = torch.Generator(device="cpu").manual_seed(31)
    q = torch.randn((B, *spatial, Hq, D), generator=g).to(dtype).cuda()
    k = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    try:
        _cabi.set_force("simt")
        ref = _backend.qk_forward(q, k, ks, dil, st, causal, D ** -0.5)
        _cabi.set_force("tc")
        got = _backend.qk_forward(q, k, ks, dil, st, causal, D ** -0.5)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    assert got.shape == ref.shape
    masked = torch.isinf(ref)
    assert torch.equal(torch.isinf(got), masked)                 # the same slots are masked (-inf)
    err = (got.float() - ref.float())[~masked].abs().max().item()
    assert err <= 2e-2 * max(1.0, ref.float()[~masked].abs().max().item()), f"logits differ by {err}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", [c for c in SPLIT_CASES if all(s == 1 for s in c[6])], ids=_split_id)
def test_tc_av_backward_matches_simt(case, dtype):
    spatial, B, Hq, Hkv, ks, dil, st, causal, D = case
    g = torch.Generator(device="cpu").manual_seed(37)
    ktot = 1
    for kk in ks:
        ktot *= kk
    attn = torch.softmax(torch.randn((B, *spatial, Hq, ktot), generator=g), dim=-1).to(dtype).cuda()
    v = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    go = torch.randn((B, *spatial, Hq, D), generator=g).to(dtype).cuda()
    try:
        _cabi.set_force("simt")
        ref_da, ref_dv = _backend.av_backward(go, attn, v, ks, dil, st, causal)
        _cabi.set_force("tc")
        da, dv = _backend.av_backward(go, attn, v, ks, dil, st, causal)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    for name, a, r in (("dattn", da, ref_da), ("dv", dv, ref_dv)):
        err = (a.float() - r.float()).abs().max().item()
        assert err <= 2e-2 * max(1.0, r.float().abs().max().item()), f"{name} differs by {err}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", SPLIT_CASES, ids=_split_id)
def test_tc_av_forward_matches_simt(case, dtype):
    spatial, B, Hq, Hkv, ks, dil, st, causal, D = case
    g = torch.Generator(device="cpu").manual_seed(41)
    ktot = 1
    for kk in ks:
        ktot *= kk
    osp = [-(-n // s) for n, s in zip(spatial, st)]
    attn = torch.softmax(torch.randn((B, *osp, Hq, ktot), generator=g), dim=-1).to(dtype).cuda()
    v = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    try:
        _cabi.set_force("simt")
        ref = _backend.av_forward(attn, v, ks, dil, st, causal)
        _cabi.set_force("tc")
        got = _backend.av_forward(attn, v, ks, dil, st, causal)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    err = (got.float() - ref.float()).abs().max().item()
    assert err <= 2e-2 * max(1.0, ref.float().abs().max().item()), f"out differs by {err}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", [c for c in SPLIT_CASES if all(s == 1 for s in c[6])], ids=_split_id)
def test_tc_qk_backward_matches_simt(case, dtype):
    spatial, B, Hq, Hkv, ks, dil, st, causal, D = case
    g = torch.Generator(device="cpu").manual_seed(43)
    ktot = 1
    for kk in ks:
        ktot *= kk
    q = torch.randn((B, *spatial, Hq, D), generator=g).to(dtype).cuda()
    k = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    dl = torch.randn((B, *spatial, Hq, ktot), generator=g).to(dtype).cuda()
    try:
        _cabi.set_force("simt")
        ref_dq, ref_dk = _backend.qk_backward(dl, q, k, ks, dil, st, causal, D ** -0.5)
        _cabi.set_force("tc")
        dq, dk = _backend.qk_backward(dl, q, k, ks, dil, st, causal, D ** -0.5)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    for name, a, r in (("dq", dq, ref_dq), ("dk", dk, ref_dk)):
        err = (a.float() - r.float()).abs().max().item()
        assert err <= 2e-2 * max(1.0, r.float().abs().max().item()), f"{name} differs by {err}"


STRIDED_BWD_CASES = [
    # spatial, B, Hq, Hkv, kernel, dilation, stride, causal, D
    ((40, 36), 1, 2, 2, (5, 5), (1, 1), (2, 2), (False, False), 64),
    ((33, 40), 2, 2, 1, (7, 3), (2, 1), (2, 3), (False, True), 64),
    ((128, 128), 1, 2, 2, (13, 13), (2, 2), (2, 2), (False, False), 64),      # the dilated benchmark shape, stride 2
    ((301,), 2, 4, 2, (31,), (1,), (4,), (False,), 128),
    ((6, 10, 12), 1, 2, 2, (3, 3, 5), (1, 1, 1), (1, 2, 2), (True, False, False), 64),
    ((30, 28), 1, 2, 2, (5, 5), (1, 1), (3, 2), (False, False), 32),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("case", STRIDED_BWD_CASES, ids=lambda c: "x".join(map(str, c[0])) + f"_s{c[6][-1]}_h{c[8]}")
def test_tc_strided_backward_matches_simt(case, dtype):
    """Output stride: the tensor-core backward runs on full-resolution copies of dout / lse / delta in
    which the rows that are not queries contribute nothing; dq must be exactly zero there."""
    spatial, B, Hq, Hkv, ks, dil, st, causal, D = case
    g = torch.Generator(device="cpu").manual_seed(19)
    osp = [-(-n // s) for n, s in zip(spatial, st)]
    q = torch.randn((B, *spatial, Hq, D), generator=g).to(dtype).cuda()
    k = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    v = torch.randn((B, *spatial, Hkv, D), generator=g).to(dtype).cuda()
    go = torch.randn((B, *osp, Hq, D), generator=g).to(dtype).cuda()
    glse = torch.randn((B, *osp, Hq), generator=g).cuda()
    geo = (ks, st, dil, causal, D ** -0.5)
    try:
        _cabi.set_force("simt")
        out, lse = _backend.fused_forward(q, k, v, *geo)
        ref = _backend.fused_backward(q, k, v, out, lse, go, *geo, dlse=glse)
        _cabi.set_force("tc")
        got = _backend.fused_backward(q, k, v, out, lse, go, *geo, dlse=glse)
        assert _cabi.last_path() == "tcgen05"
    finally:
        _cabi.set_force(None)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    for name, a, r in zip(("dq", "dk", "dv"), got[:3], ref[:3]):
        err = (a.float() - r.float()).abs().max().item()
        scale = max(1.0, r.float().abs().max().item())
        assert err <= 2e-2 * scale, f"{name} differs by {err} (scale {scale})"
    # positions that are not queries get exactly zero dq
    mask = torch.ones(spatial, dtype=torch.bool)
    mask[tuple(slice(None, None, s) for s in st)] = False
    assert float(got[0][:, mask.cuda()].abs().sum()) == 0.0
