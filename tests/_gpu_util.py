"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import oracle
from natten_mps_b200 import functional as F

FUSED = {1: F.na1d, 2: F.na2d, 3: F.na3d}
QK = {1: F.na1d_qk, 2: F.na2d_qk, 3: F.na3d_qk}
AV = {1: F.na1d_av, 2: F.na2d_av, 3: F.na3d_av}
VARLEN = {1: F.na1d_varlen, 2: F.na2d_varlen, 3: F.na3d_varlen}

# Parity contract: 1e-5 relative in float32; 2e-2 absolute for bf16/fp16 against a
# float32-or-better reference on the same (already rounded) inputs.
TOL = {torch.float64: 1e-10, torch.float32: 1e-5, torch.float16: 2e-2, torch.bfloat16: 2e-2}


def dev(a, dtype, grad=False):
    t = torch.as_tensor(np.asarray(a)).to(dtype).cuda()
    return t.requires_grad_(True) if grad else t


def rounded(a, dtype):
    """The values the GPU actually sees, as float64 numpy (inputs rounded to dtype)."""
    return torch.as_tensor(np.asarray(a)).to(dtype).double().numpy()


def check(name, got, want, dtype, scale_rel=False):
    """``scale_rel``: measure 16-bit results relative to the tensor's magnitude.  Used for the
    split ops, whose raw (unscaled) logits reach |q||k| ~ 10: one bf16 ulp there is 0.03, so the
    output format alone exceeds an absolute 2e-2."""
    got = got.detach().double().cpu().numpy()
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    fg, fw = np.isfinite(got), np.isfinite(want)
    assert np.array_equal(fg, fw), f"{name}: finite pattern differs"
    assert np.array_equal(got[~fg], want[~fw]), f"{name}: inf pattern differs"
    if not fw.any():
        return 0.0
    err = float(np.abs(got[fg] - want[fw]).max())
    tol = TOL[dtype]
    if dtype in (torch.float32, torch.float64) or scale_rel:
        tol = tol * max(1.0, float(np.abs(want[fw]).max()))     # relative to the tensor's scale
    assert err <= tol, f"{name}: max abs err {err:.3e} > {tol:.3e} ({dtype})"
    return err


def run_fused(rank, dtype, q, k, v, gout, kwargs, ek=None, ev=None, glse=None, sizes=None):
    """Run the CUDA path (forward + autograd backward) and the float64 oracle on the
    same rounded inputs; returns two dicts of results."""
    kw = dict(kwargs)
    want_lse = kw.pop("return_lse", False) or glse is not None
    qd, kd, vd = dev(q, dtype, True), dev(k, dtype, True), dev(v, dtype, True)
    leaves = [qd, kd, vd]
    extra = {}
    if ek is not None:
        ekd, evd = dev(ek, dtype, True), dev(ev, dtype, True)
        extra = dict(additional_keys=ekd, additional_values=evd)
        leaves += [ekd, evd]
    if sizes is not None:
        st = torch.tensor(sizes, dtype=torch.int32).cuda()
        out = VARLEN[rank](qd, kd, vd, st[:, 0] if rank == 1 else st, **kw, **extra)
        lse = None
    elif want_lse:
        out, lse = FUSED[rank](qd, kd, vd, return_lse=True, **kw, **extra)
    else:
        out, lse = FUSED[rank](qd, kd, vd, **kw, **extra), None
    loss = (out.double() * dev(gout, torch.float64)).sum()
    if glse is not None:
        loss = loss + (lse.double() * dev(glse, torch.float64)).sum()
    grads = torch.autograd.grad(loss, leaves)
    got = dict(out=out, lse=lse, dq=grads[0], dk=grads[1], dv=grads[2])
    if ek is not None:
        got.update(dek=grads[3], dev=grads[4])

    r = lambda a: None if a is None else rounded(a, dtype)
    okw = dict(kw)
    okw.update(additional_keys=r(ek), additional_values=r(ev), extents=sizes)
    ref_out, ref_lse = oracle.na_forward(r(q), r(k), r(v), **okw)
    # gradient of the loss as autograd sees it: dout (and dlse) in float64
    rg = oracle.na_backward(r(q), r(k), r(v), ref_out, ref_lse, np.asarray(gout, dtype=np.float64),
                            dlse=None if glse is None else np.asarray(glse, dtype=np.float64), **okw)
    want = dict(out=ref_out, lse=ref_lse, dq=rg[0], dk=rg[1], dv=rg[2], dek=rg[3], dev=rg[4])
    return got, want


def compare_fused(got, want, dtype, grads_of_rounded_dout=True):
    errs = {}
    for name in ("out", "lse", "dq", "dk", "dv", "dek", "dev"):
        if got.get(name) is not None and want.get(name) is not None:
            errs[name] = check(name, got[name], want[name], dtype)
    return errs
