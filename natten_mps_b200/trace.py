"""Clock-stamp timeline of one CTA of each tensor-core kernel.

    python -m natten_mps_b200.trace [--batch 8]

Runs config-2-shaped forward and backward calls with ``natten_debug_trace`` armed and
prints, for CTA (5, 0, 0) of each kernel, the cycles between pipeline events: for the
issuing thread (loads landed -> first MMAs issued -> per chunk: threads done / MMAs
issued) and for softmax / compute warp 0 (per chunk: wait for scores, work, publish).
Useful to see whether a change shortens the per-chunk dependency chain.
"""
from __future__ import annotations

import argparse
import ctypes

import torch

from . import _backend, _cabi


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    args = ap.parse_args()
    torch.manual_seed(0)
    q, k, v, go = [torch.randn(args.batch, 64, 64, 8, 64, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    geo = ((7, 7), (1, 1), (1, 1), (False, False), 0.125)
    out, lse = _backend.fused_forward(q, k, v, *geo)
    for _ in range(3):
        _backend.fused_forward(q, k, v, *geo)
        _backend.fused_backward(q, k, v, out, lse, go, *geo)
    buf = torch.zeros(512, dtype=torch.int64, device="cuda")
    lib = _cabi.lib()
    lib.natten_debug_trace.argtypes = [ctypes.c_void_p]
    lib.natten_debug_trace(ctypes.c_void_p(buf.data_ptr()))
    _backend.fused_forward(q, k, v, *geo)
    _backend.fused_backward(q, k, v, out, lse, go, *geo)
    torch.cuda.synchronize()
    lib.natten_debug_trace(None)
    t = buf.cpu().tolist()
    for name, base in (("forward, issuing thread", 256), ("forward, softmax warp 0", 320),
                       ("backward query side, issuing thread", 0), ("backward query side, compute warp 0", 64),
                       ("backward key side, issuing thread", 128), ("backward key side, compute warp 0", 192)):
        xs = [x for x in t[base:base + 56] if x]
        print(f"{name}: {len(xs)} stamps, deltas (cycles): {[xs[i + 1] - xs[i] for i in range(len(xs) - 1)]}")
    print("forward CTA lifetime (cycles):", t[256 + 121] - t[256 + 120])


if __name__ == "__main__":
    main()
