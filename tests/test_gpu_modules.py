"""``NeighborhoodAttention{1,2,3}D`` against fixtures produced by the reference's own modules
(``src/natten_mps/nn/na1d.py:60-125``, ``na2d.py:88-122``, ``na3d.py``): the reference module's
``state_dict`` is loaded into the module of this package, the stored input goes in, and the
output, the input gradient and every parameter gradient must match.

float64 runs the exact-arithmetic kernels (1e-9 relative to each tensor's magnitude); bf16 runs the
projections in bf16 and the attention on tensor cores or the 16-bit kernels (2e-2 absolute on the
output and input gradient; parameter gradients are sums over every token, so they are measured
relative to the tensor's largest entry)."""
import numpy as np
import pytest
import torch

import natten_mps_b200 as nb
from tests import _golden as G

pytestmark = pytest.mark.gpu


def _tuple_ctor(ctor):
    return {k: (tuple(v) if isinstance(v, list) else v) for k, v in ctor.items()}


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.bfloat16], ids=["f64", "f32", "bf16"])
@pytest.mark.parametrize("case", G.module_cases(), ids=lambda c: c["name"])
def test_module_matches_reference_module(case, dtype):
    a = G.arrays(case["name"])
    m = getattr(nb, case["cls"])(**_tuple_ctor(case["ctor"]))
    state = {k[2:]: torch.as_tensor(v) for k, v in a.items() if k.startswith("p.")}
    assert set(state) == set(m.state_dict()), "parameter names differ from the reference module"
    m.load_state_dict(state)
    m = m.to(device="cuda", dtype=dtype)
    x = torch.as_tensor(a["x"]).to(dtype).cuda().requires_grad_(True)
    y = m(x)
    assert tuple(y.shape) == a["y"].shape
    params = dict(m.named_parameters())
    grads = torch.autograd.grad((y.double() * torch.as_tensor(a["gout"]).cuda()).sum(), [x] + list(params.values()))

    def close(name, got, want, tol, rel):
        got = got.detach().double().cpu().numpy()
        err = float(np.abs(got - want).max())
        bound = tol * (max(1.0, float(np.abs(want).max())) if rel else 1.0)
        print(f"  {case['name']} {name}: max-abs {err:.3e} (bound {bound:.3e}, max|want| {np.abs(want).max():.2f})")
        assert err <= bound, (name, err, bound)

    if dtype == torch.bfloat16:
        close("y", y, a["y"], 2e-2, False)
        close("dx", grads[0], a["dx"], 2e-2, False)
        for (pn, _), g in zip(params.items(), grads[1:]):
            close("d" + pn, g, a["dp." + pn], 3e-2, True)
    else:
        tol = 1e-9 if dtype == torch.float64 else 2e-5
        close("y", y, a["y"], tol, True)
        close("dx", grads[0], a["dx"], tol, True)
        for (pn, _), g in zip(params.items(), grads[1:]):
            close("d" + pn, g, a["dp." + pn], tol, True)
