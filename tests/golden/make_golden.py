"""Generate the golden fixtures in this folder from the reference itself.

Run once, in a container that has the reference checkout:

    NATTEN_BACKEND=pure PYTHONPATH=<reference>/src python tests/golden/make_golden.py

It imports the reference package unchanged (its pure-PyTorch backend), runs the
cases below in float64 on CPU and writes ``golden.npz`` + ``golden.json`` next
to this file.  The fixtures travel with the repository; the reference does not
have to be present to run the tests.

Inputs are drawn with ``torch.Generator().manual_seed(seed)`` in the order
q, k, v, grad_out, (additional_keys, additional_values), (grad_lse) and are
stored in the fixture, so the tests do not depend on torch's RNG stream.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

os.environ.setdefault("NATTEN_BACKEND", "pure")
import natten_mps  # noqa: E402  (the reference package)
from natten_mps import functional as RF  # noqa: E402
from natten_mps.utils.window import get_window_start  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
assert natten_mps.get_backend() == "pure"

FUSED = [
    # name, rank, spatial, B, Hq, Hkv, D, kwargs
    ("na1d_basic", 1, (32,), 2, 2, 2, 8, dict(kernel_size=7)),
    ("na1d_config1", 1, (128,), 2, 4, 4, 32, dict(kernel_size=7)),
    ("na1d_dil", 1, (24,), 2, 2, 2, 8, dict(kernel_size=5, dilation=2)),
    ("na1d_dil3_ragged", 1, (23,), 1, 2, 2, 4, dict(kernel_size=3, dilation=3)),
    ("na1d_causal", 1, (20,), 2, 2, 2, 8, dict(kernel_size=5, is_causal=True)),
    ("na1d_stride", 1, (21,), 2, 2, 2, 8, dict(kernel_size=5, stride=2)),
    ("na1d_all", 1, (26,), 1, 2, 2, 8, dict(kernel_size=4, stride=3, dilation=2, is_causal=True)),
    ("na1d_evenk", 1, (19,), 1, 2, 2, 8, dict(kernel_size=4)),
    ("na1d_gqa", 1, (18,), 2, 4, 2, 8, dict(kernel_size=5)),
    ("na1d_mqa_scale", 1, (18,), 1, 4, 1, 8, dict(kernel_size=3, scale=0.3)),
    ("na1d_extra", 1, (16,), 2, 4, 2, 8, dict(kernel_size=5), 3),
    ("na1d_lse", 1, (16,), 2, 2, 2, 8, dict(kernel_size=5, return_lse=True)),
    ("na1d_extra_lse", 1, (16,), 2, 2, 2, 8, dict(kernel_size=3, dilation=2, return_lse=True), 2),
    ("na2d_basic", 2, (10, 12), 2, 2, 2, 8, dict(kernel_size=(3, 5))),
    ("na2d_k7", 2, (9, 11), 1, 2, 2, 16, dict(kernel_size=7)),
    ("na2d_dil", 2, (12, 9), 1, 2, 2, 8, dict(kernel_size=(3, 3), dilation=(3, 2))),
    ("na2d_causal_stride", 2, (9, 10), 1, 2, 2, 8,
     dict(kernel_size=(3, 5), stride=(2, 1), is_causal=(True, False))),
    ("na2d_stride_dil", 2, (13, 12), 1, 2, 2, 8, dict(kernel_size=5, stride=2, dilation=2)),
    ("na2d_gqa_extra", 2, (8, 8), 2, 4, 2, 8, dict(kernel_size=3), 4),
    ("na3d_basic", 3, (5, 6, 7), 1, 2, 2, 8, dict(kernel_size=(3, 3, 5))),
    ("na3d_causal_d", 3, (6, 7, 7), 1, 2, 2, 8,
     dict(kernel_size=(3, 5, 5), is_causal=(True, False, False))),
    ("na3d_mixed", 3, (6, 6, 8), 1, 2, 1, 4,
     dict(kernel_size=(3, 3, 3), stride=(1, 2, 1), dilation=(1, 1, 2), is_causal=(False, False, True))),
]

SPLIT = [
    ("qk1d", 1, (17,), 2, 2, 8, dict(kernel_size=5)),
    ("qk1d_scale_causal", 1, (17,), 1, 2, 8, dict(kernel_size=5, is_causal=True, scale=0.25)),
    ("qk1d_stride_dil", 1, (22,), 1, 2, 8, dict(kernel_size=3, dilation=3, stride=2)),
    ("qk2d", 2, (8, 9), 1, 2, 8, dict(kernel_size=(3, 5))),
    ("qk2d_causal_stride", 2, (8, 9), 1, 2, 8,
     dict(kernel_size=3, stride=(2, 2), is_causal=(False, True), scale=0.5)),
    ("qk3d", 3, (4, 5, 6), 1, 2, 4, dict(kernel_size=3, dilation=(1, 1, 2))),
    # head dims that reach the vectorised 16-bit kernels and the tensor-core kernels (D_v == D here)
    ("qk2d_d32", 2, (10, 9), 1, 2, 32, dict(kernel_size=(5, 3)), 32),
    ("qk2d_d64_dil_scale", 2, (12, 11), 1, 2, 64, dict(kernel_size=3, dilation=(2, 1), scale=0.125), 64),
]

# Module fixtures: constructor of the reference module, input shape.  The state_dict, the input,
# the output, the input gradient and every parameter gradient are stored.
MODULES = [
    ("mod2d", "NeighborhoodAttention2D", dict(embed_dim=64, num_heads=2, kernel_size=5), (2, 10, 12, 64)),
    ("mod1d_gqa", "NeighborhoodAttention1D", dict(embed_dim=64, num_heads=4, kernel_size=5, num_kv_heads=2),
     (2, 20, 64)),
    ("mod3d_causal_stride", "NeighborhoodAttention3D",
     dict(embed_dim=32, num_heads=2, kernel_size=(3, 3, 3), stride=(1, 2, 1), is_causal=(True, False, False),
          qk_scale=0.2), (1, 4, 6, 6, 32)),
]

# Relative position bias (compat.v014 operators, heads-first there; stored heads-last here).
RPB = [
    ("rpb1d", 1, (19,), 2, 2, 8, dict(kernel_size=5, dilation=1)),
    ("rpb1d_dil", 1, (23,), 1, 3, 4, dict(kernel_size=3, dilation=3)),
    ("rpb2d", 2, (9, 8), 1, 2, 8, dict(kernel_size=(3, 5), dilation=(1, 1))),
    ("rpb2d_dil_d32", 2, (14, 12), 1, 2, 32, dict(kernel_size=(5, 3), dilation=(2, 3))),
]

VARLEN = [
    ("var1d", 1, (20,), 3, 2, 8, dict(kernel_size=5), [[20], [7], [12]]),
    ("var1d_dil", 1, (24,), 2, 2, 8, dict(kernel_size=3, dilation=2), [[24], [9]]),
    ("var2d", 2, (9, 10), 2, 2, 8, dict(kernel_size=3), [[9, 10], [5, 7]]),
    ("var3d", 3, (5, 6, 6), 2, 2, 4, dict(kernel_size=3), [[5, 6, 6], [3, 4, 5]]),
]


def _randn(g, *shape):
    # drawn in float32 (so the fixture stores inputs exactly as float32), computed in float64
    return torch.randn(*shape, generator=g, dtype=torch.float32).double()


def main():
    arrays = {}
    manifest = {"fused": [], "split": [], "varlen": [], "modules": [], "rpb": [], "window": None}
    fns = {1: RF.na1d, 2: RF.na2d, 3: RF.na3d}
    qk = {1: RF.na1d_qk, 2: RF.na2d_qk, 3: RF.na3d_qk}
    av = {1: RF.na1d_av, 2: RF.na2d_av, 3: RF.na3d_av}
    var = {1: RF.na1d_varlen, 2: RF.na2d_varlen, 3: RF.na3d_varlen}

    for seed, case in enumerate(FUSED):
        name, rank, spatial, B, Hq, Hkv, D, kwargs = case[:8]
        n_extra = case[8] if len(case) > 8 else 0
        g = torch.Generator().manual_seed(seed)
        q = _randn(g, B, *spatial, Hq, D).requires_grad_()
        k = _randn(g, B, *spatial, Hkv, D).requires_grad_()
        v = _randn(g, B, *spatial, Hkv, D).requires_grad_()
        kw = dict(kwargs)
        leaves = [q, k, v]
        if n_extra:
            ek = _randn(g, B, n_extra, Hkv, D).requires_grad_()
            ev = _randn(g, B, n_extra, Hkv, D).requires_grad_()
            kw.update(additional_keys=ek, additional_values=ev)
            leaves += [ek, ev]
        res = fns[rank](q, k, v, **kw)
        out, lse = res if isinstance(res, tuple) else (res, None)
        gout = _randn(g, *out.shape)
        loss = (out * gout).sum()
        if lse is not None:
            glse = _randn(g, *lse.shape)
            loss = loss + (lse.double() * glse).sum()
            arrays[f"{name}/glse"] = glse.numpy()
            arrays[f"{name}/lse"] = lse.detach().double().numpy()
        grads = torch.autograd.grad(loss, leaves)
        for nm, t in zip(["q", "k", "v", "ek", "ev"], leaves):
            arrays[f"{name}/{nm}"] = t.detach().numpy()
        for nm, t in zip(["dq", "dk", "dv", "dek", "dev"], grads):
            arrays[f"{name}/{nm}"] = t.numpy()
        arrays[f"{name}/out"] = out.detach().numpy()
        arrays[f"{name}/gout"] = gout.numpy()
        manifest["fused"].append(dict(name=name, rank=rank, kwargs=kwargs, n_extra=n_extra))

    for seed, case in enumerate(SPLIT, start=100):
        name, rank, spatial, B, H, D, kwargs = case[:7]
        Dv = case[7] if len(case) > 7 else D + 4                 # D_v != D_qk is legal here
        g = torch.Generator().manual_seed(seed)
        q = _randn(g, B, *spatial, H, D).requires_grad_()
        k = _randn(g, B, *spatial, H, D).requires_grad_()
        v = _randn(g, B, *spatial, H, Dv).requires_grad_()
        logits = qk[rank](q, k, **kwargs)
        glog = _randn(g, *logits.shape)
        finite = torch.isfinite(logits)
        dq, dk = torch.autograd.grad((torch.where(finite, logits, 0.0) * glog).sum(), [q, k])
        attn = _randn(g, *logits.shape).requires_grad_()          # any real weights
        av_kwargs = {k_: v_ for k_, v_ in kwargs.items() if k_ != "scale"}
        out = av[rank](attn, v, **av_kwargs)
        gout = _randn(g, *out.shape)
        dattn, dv = torch.autograd.grad((out * gout).sum(), [attn, v])
        for nm, t in dict(q=q, k=k, v=v, logits=logits, glog=glog, dq=dq, dk=dk, attn=attn,
                          out=out, gout=gout, dattn=dattn, dv=dv).items():
            arrays[f"{name}/{nm}"] = t.detach().numpy()
        manifest["split"].append(dict(name=name, rank=rank, kwargs=kwargs))

    for seed, (name, rank, spatial, B, H, D, kwargs, sizes) in enumerate(VARLEN, start=200):
        g = torch.Generator().manual_seed(seed)
        q = _randn(g, B, *spatial, H, D).requires_grad_()
        k = _randn(g, B, *spatial, H, D).requires_grad_()
        v = _randn(g, B, *spatial, H, D).requires_grad_()
        st = torch.tensor(sizes, dtype=torch.int32)
        out = var[rank](q, k, v, st[:, 0] if rank == 1 else st, **kwargs)
        gout = _randn(g, *out.shape)
        dq, dk, dv = torch.autograd.grad((out * gout).sum(), [q, k, v])
        for nm, t in dict(q=q, k=k, v=v, out=out, gout=gout, dq=dq, dk=dk, dv=dv).items():
            arrays[f"{name}/{nm}"] = t.detach().numpy()
        manifest["varlen"].append(dict(name=name, rank=rank, kwargs=kwargs, sizes=sizes))

    for seed, (name, cls, ctor, xshape) in enumerate(MODULES, start=300):
        torch.manual_seed(seed)
        m = getattr(natten_mps, cls)(**ctor).double()            # float32-initialised parameters, float64 maths
        g = torch.Generator().manual_seed(seed)
        x = _randn(g, *xshape).requires_grad_()
        y = m(x)
        gout = _randn(g, *y.shape)
        params = dict(m.named_parameters())
        grads = torch.autograd.grad((y * gout).sum(), [x] + list(params.values()))
        arrays[f"{name}/x"] = x.detach().numpy()
        arrays[f"{name}/gout"] = gout.numpy()
        arrays[f"{name}/y"] = y.detach().numpy()
        arrays[f"{name}/dx"] = grads[0].numpy()
        for (pn, pt), gt in zip(params.items(), grads[1:]):
            arrays[f"{name}/p.{pn}"] = pt.detach().numpy()
            arrays[f"{name}/dp.{pn}"] = gt.numpy()
        manifest["modules"].append(dict(name=name, cls=cls, ctor=ctor))

    from natten_mps.compat import v014 as C14
    from natten_mps.utils.window import get_pb_start
    for seed, (name, rank, spatial, B, H, D, kwargs) in enumerate(RPB, start=400):
        g = torch.Generator().manual_seed(seed)
        ks = kwargs["kernel_size"] if isinstance(kwargs["kernel_size"], tuple) else (kwargs["kernel_size"],)
        q = _randn(g, B, *spatial, H, D).requires_grad_()
        k = _randn(g, B, *spatial, H, D).requires_grad_()
        rpb = _randn(g, H, *[2 * x - 1 for x in ks]).requires_grad_()
        if rank == 1:
            logits = C14.natten1dqkrpb(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), rpb,
                                       kwargs["kernel_size"], kwargs["dilation"]).permute(0, 2, 1, 3)
        else:
            logits = C14.natten2dqkrpb(q.permute(0, 3, 1, 2, 4), k.permute(0, 3, 1, 2, 4), rpb,
                                       kwargs["kernel_size"], kwargs["dilation"]).permute(0, 2, 3, 1, 4)
        glog = _randn(g, *logits.shape)
        dq, dk, drpb = torch.autograd.grad((logits * glog).sum(), [q, k, rpb])
        for nm, t in dict(q=q, k=k, rpb=rpb, logits=logits, glog=glog, dq=dq, dk=dk, drpb=drpb).items():
            arrays[f"{name}/{nm}"] = t.detach().contiguous().numpy()
        manifest["rpb"].append(dict(name=name, rank=rank, kwargs=kwargs))
    pb_rows = []
    for L in range(1, 41):
        for K in range(1, 12):
            for dil in range(1, 5):
                if K * dil > L:
                    continue
                for i in range(L):
                    pb_rows.append(get_pb_start(i, L, K, dil))
    arrays["window/pb_start"] = np.asarray(pb_rows, dtype=np.int16)

    # integer spec: every legal (L, K, dilation) with L <= 40, K <= 11, dilation <= 4
    rows = []
    for L in range(1, 41):
        for K in range(1, 12):
            for dil in range(1, 5):
                if K * dil > L:
                    continue
                for i in range(L):
                    rows.append(get_window_start(i, L, K, dil))
    arrays["window/start"] = np.asarray(rows, dtype=np.int16)
    manifest["window"] = dict(rows=len(rows), order="for L in 1..40: for K in 1..11: for dil in 1..4 "
                              "(skip K*dil > L): for index in 0..L-1")

    def _json(o):
        if isinstance(o, tuple):
            return list(o)
        raise TypeError(type(o))

    inputs = {"q", "k", "v", "ek", "ev", "gout", "glse", "glog", "attn", "x", "rpb"}

    def _store(key, a):
        if a.dtype == np.int16:
            return a
        if key.split("/")[1] in inputs or key.split("/")[1].startswith("p."):
            assert np.array_equal(a.astype(np.float32).astype(np.float64), a)
            return a.astype(np.float32)
        return a.astype(np.float64)

    np.savez_compressed(os.path.join(HERE, "golden.npz"), **{k_: _store(k_, a) for k_, a in arrays.items()})
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(manifest, f, indent=1, default=_json)
    print("wrote", len(arrays), "arrays;", sum(a.nbytes for a in arrays.values()) / 1e6, "MB raw")


if __name__ == "__main__":
    sys.exit(main())
