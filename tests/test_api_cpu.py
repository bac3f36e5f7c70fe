"""Host-side logic that needs no GPU: validation, shape functions, the C ABI's
exported symbols, the window arithmetic and the merge helper."""
import ctypes
import os
import re

import pytest
import torch

import natten_mps_b200 as nb
from natten_mps_b200 import _cabi, functional as F, merge_attentions
from natten_mps_b200.utils import get_window_start, get_window_start_vectorized
from tests import _golden as G

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "natten_b200.h")).read()
    declared = set(re.findall(r"\b(natten_[a-z0-9_]+)\s*\(", header))
    declared -= {"natten_params_t"}
    assert declared == set(_cabi.EXPORTS)
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.natten_abi_version() == 1
    lib.natten_strerror.restype = ctypes.c_char_p
    assert lib.natten_strerror(-2) == b"unsupported configuration"


def test_params_are_checked_without_a_gpu():
    L = _cabi.lib()
    p = _cabi.make_params(1, torch.float32, 1, 2, 2, 8, 8, (16,), (5,), (1,), (1,), (False,), 0.5)
    p.rank = 4
    assert L.natten_fused_fwd(p, *([None] * 8)) == -1
    p.rank = 1
    p.kernel[0] = 17                       # kernel > extent
    assert L.natten_fused_fwd(p, *([None] * 8)) == -1
    p.kernel[0] = 5
    p.heads_q, p.heads_kv = 3, 2           # not divisible
    assert L.natten_fused_fwd(p, *([None] * 8)) == -1
    p.heads_q = 4
    p.dim = 512
    assert L.natten_fused_fwd(p, *([None] * 8)) == -2
    with pytest.raises(NotImplementedError):
        _cabi.check(-2, "x")
    with pytest.raises(ValueError):
        _cabi.check(-1, "x")


def test_workspace_size():
    p = _cabi.make_params(2, torch.bfloat16, 2, 4, 2, 64, 64, (16, 16), (3, 3), (1, 1), (1, 1),
                          (False, False), 0.125)
    n = _cabi.lib().natten_workspace_bytes(p, _cabi.OP_FUSED_BWD)
    assert n >= 2 * 16 * 16 * 4 * 4 and n % 256 == 0


def test_window_start_matches_reference_table():
    for i, L, K, dil, start in G.window_rows():
        assert get_window_start(i, L, K, dil) == start
    for L, K, dil in [(17, 5, 1), (23, 3, 3), (12, 4, 2), (40, 11, 3)]:
        idx = torch.arange(L)
        vec = get_window_start_vectorized(idx, L, K, dil).tolist()
        assert vec == [get_window_start(i, L, K, dil) for i in range(L)]


def _meta(*shape):
    return torch.empty(*shape, device="meta")


def test_shapes_via_meta_tensors():
    q = _meta(2, 17, 4, 8)
    assert F.na1d(q, q, q, 5, stride=2).shape == (2, 9, 4, 8)
    out, lse = F.na1d(q, _meta(2, 17, 2, 8), _meta(2, 17, 2, 8), 5, return_lse=True)
    assert out.shape == (2, 17, 4, 8) and lse.shape == (2, 17, 4)
    q2 = _meta(1, 9, 10, 2, 16)
    assert F.na2d(q2, q2, q2, (3, 5), stride=(2, 3)).shape == (1, 5, 4, 2, 16)
    assert F.na2d_qk(q2, q2, (3, 5)).shape == (1, 9, 10, 2, 15)
    assert F.na2d_av(_meta(1, 9, 10, 2, 15), _meta(1, 9, 10, 2, 24), (3, 5)).shape == (1, 9, 10, 2, 24)
    q3 = _meta(1, 4, 5, 6, 2, 8)
    assert F.na3d(q3, q3, q3, 3).shape == q3.shape
    assert F.na3d_qk(q3, q3, 3, stride=2).shape == (1, 2, 3, 3, 2, 27)
    assert torch.ops.natten_b200.na2d_fwd(q2, q2, q2, [3, 3], [1, 1], [1, 1], [False, False], None).shape == q2.shape


def test_validation_errors():
    q = _meta(2, 16, 4, 8)
    with pytest.raises(ValueError, match="expects query/key/value"):
        F.na1d(_meta(2, 16, 8), q, q, 3)
    with pytest.raises(ValueError, match="Spatial"):
        F.na1d(q, _meta(2, 15, 4, 8), q, 3)
    with pytest.raises(ValueError, match="Head dim"):
        F.na1d(q, _meta(2, 16, 4, 4), q, 3)
    with pytest.raises(ValueError, match="divisible"):
        F.na1d(q, _meta(2, 16, 3, 8), _meta(2, 16, 3, 8), 3)
    with pytest.raises(ValueError, match="cannot exceed"):
        F.na1d(q, q, q, 17)
    with pytest.raises(ValueError, match="stride"):
        F.na1d(q, q, q, 3, stride=4)
    with pytest.raises(ValueError, match="exceeds input"):
        F.na1d(q, q, q, 5, dilation=4)
    with pytest.raises(ValueError, match="> 0"):
        F.na1d(q, q, q, 0)
    with pytest.raises(ValueError, match="length 2"):
        F.na2d(_meta(1, 8, 8, 2, 4), _meta(1, 8, 8, 2, 4), _meta(1, 8, 8, 2, 4), (3, 3, 3))
    with pytest.raises(ValueError, match="both be provided"):
        F.na1d(q, q, q, 3, additional_keys=_meta(2, 3, 4, 8))
    with pytest.raises(ValueError, match="4D"):
        F.na1d(q, q, q, 3, additional_keys=_meta(2, 3, 8), additional_values=_meta(2, 3, 8))
    with pytest.raises(ValueError, match="batch"):
        F.na1d(q, q, q, 3, additional_keys=_meta(1, 3, 4, 8), additional_values=_meta(1, 3, 4, 8))
    with pytest.raises(ValueError, match="head dim"):
        F.na1d(q, q, q, 3, additional_keys=_meta(2, 3, 4, 4), additional_values=_meta(2, 3, 4, 4))
    with pytest.raises(ValueError, match="same shape"):
        F.na1d_qk(q, _meta(2, 16, 2, 8), 3)
    with pytest.raises(ValueError, match="must match kernel_size"):
        F.na1d_av(_meta(2, 16, 4, 5), q, 3)
    with pytest.raises(ValueError, match="kernel_size"):
        F.na1d_varlen(q, q, q, torch.tensor([16, 2]), 3)
    with pytest.raises(ValueError, match="L_max"):
        F.na1d_varlen(q, q, q, torch.tensor([16, 17]), 3)
    with pytest.raises(ValueError, match="int32 or int64"):
        F.na1d_varlen(q, q, q, torch.tensor([16.0, 12.0]), 3)
    with pytest.raises(ValueError, match=r"\[B, 2\]"):
        F.na2d_varlen(_meta(2, 8, 8, 2, 4), _meta(2, 8, 8, 2, 4), _meta(2, 8, 8, 2, 4), torch.tensor([8, 8]), 3)


def test_cpu_tensors_are_rejected_not_emulated():
    q = torch.randn(1, 8, 2, 4)
    with pytest.raises((NotImplementedError, RuntimeError)):
        F.na1d(q, q, q, 3)


def test_backend_shims_and_support_matrix():
    assert nb.get_backend() == "cuda"
    nb.set_backend("auto")
    nb.set_backend("cuda")
    with pytest.raises(NotImplementedError):
        nb.set_backend("metal")
    m = nb.get_support_matrix()
    assert set(m) == {"cuda"} and m["cuda"]["fusion"]["na2d"] is True


def test_merge_attentions_equals_joint_softmax():
    torch.manual_seed(0)
    s = torch.randn(2, 5, 3, 11, dtype=torch.float64)
    v = torch.randn(2, 5, 3, 11, 4, dtype=torch.float64)
    parts = [(0, 4), (4, 9), (9, 11)]
    outs, lses = [], []
    for a, b in parts:
        w = torch.softmax(s[..., a:b], -1)
        outs.append((w.unsqueeze(-1) * v[..., a:b, :]).sum(-2))
        lses.append(torch.logsumexp(s[..., a:b], -1))
    out, lse = merge_attentions(outs, lses)
    want = (torch.softmax(s, -1).unsqueeze(-1) * v).sum(-2)
    assert torch.allclose(out, want, atol=1e-12)
    assert torch.allclose(lse, torch.logsumexp(s, -1), atol=1e-12)
    with pytest.raises(ValueError):
        merge_attentions(outs[:1], lses[:1])
    with pytest.raises(ValueError):
        merge_attentions(outs, lses[:2])


def test_module_parameter_names_match_the_reference_layout():
    m = nb.NeighborhoodAttention2D(32, 4, 3)
    assert set(dict(m.named_parameters())) == {"qkv.weight", "qkv.bias", "proj.weight", "proj.bias"}
    g = nb.NeighborhoodAttention1D(32, 4, 3, num_kv_heads=2, qkv_bias=False)
    assert set(dict(g.named_parameters())) == {"q_proj.weight", "kv_proj.weight", "proj.weight", "proj.bias"}
    with pytest.raises(ValueError):
        nb.NeighborhoodAttention3D(30, 4, 3)
    x = torch.empty(2, 8, 8, 32, device="meta")
    assert m.to("meta")(x).shape == (2, 8, 8, 32)


def test_host_step_needs_cuda_and_validates():
    import torch
    from natten_mps_b200.host_step import HostStep
    with pytest.raises(ValueError):
        HostStep(4, 3)
    with pytest.raises(ValueError):
        HostStep(2, 3, stride=5)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            HostStep(2, 3)


def test_module_state_dict_names_and_shapes_match_the_reference_fixture():
    """The fixture stores the reference modules' parameters; the modules here must accept them."""
    for case in G.module_cases():
        a = G.arrays(case["name"])
        ctor = {k: (tuple(v) if isinstance(v, list) else v) for k, v in case["ctor"].items()}
        m = getattr(nb, case["cls"])(**ctor)
        state = {k[2:]: torch.as_tensor(v) for k, v in a.items() if k.startswith("p.")}
        assert {k: tuple(v.shape) for k, v in state.items()} == {k: tuple(v.shape) for k, v in m.state_dict().items()}
        m.load_state_dict(state)
