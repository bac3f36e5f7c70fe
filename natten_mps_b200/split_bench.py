"""Timing of the split operators (QK / AV, forward and backward) on benchmark-shaped inputs.

    python -m natten_mps_b200.split_bench [--config c2|c3|c4|1d] [--iters 20]

Prints CUDA-event time per call and the algorithmic bandwidth (every tensor touched once at its
storage width) beside the path that ran.  The fused operator is the headline; this is the same
measurement for the two-step path (`na*_qk` -> softmax -> `na*_av`).
"""
from __future__ import annotations

import argparse

import torch

from . import _backend, _cabi

CONFIGS = {
    "c2": dict(shape=(8, 64, 64, 8, 64), kernel=(7, 7), dilation=(1, 1), causal=(False, False)),
    "c3": dict(shape=(4, 128, 128, 8, 64), kernel=(13, 13), dilation=(2, 2), causal=(False, False)),
    "c4": dict(shape=(2, 16, 32, 32, 8, 64), kernel=(3, 7, 7), dilation=(1, 1, 1), causal=(True, False, False)),
    "1d": dict(shape=(8, 4096, 8, 64), kernel=(63,), dilation=(1,), causal=(False,)),
}


def _time(fn, iters):
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    ks, dil, causal = cfg["kernel"], cfg["dilation"], cfg["causal"]
    st = (1,) * len(ks)
    g = torch.Generator(device="cpu").manual_seed(0)
    q, k, v, go = [torch.randn(cfg["shape"], generator=g).to(dtype).cuda() for _ in range(4)]
    logits = _backend.qk_forward(q, k, ks, dil, st, causal, None)
    attn = torch.softmax(logits.float(), -1).to(dtype)
    dl = torch.randn(logits.shape, generator=g).to(dtype).cuda()
    nq = q.numel() * q.element_size()
    nl = logits.numel() * logits.element_size()
    rows = [
        ("qk_fwd", lambda: _backend.qk_forward(q, k, ks, dil, st, causal, None), 2 * nq + nl),
        ("qk_bwd", lambda: _backend.qk_backward(dl, q, k, ks, dil, st, causal, None), 4 * nq + nl),
        ("av_fwd", lambda: _backend.av_forward(attn, v, ks, dil, st, causal), 2 * nq + nl),
        ("av_bwd", lambda: _backend.av_backward(go, attn, v, ks, dil, st, causal), 3 * nq + 2 * nl),
    ]
    for name, fn, nbytes in rows:
        ms = _time(fn, args.iters)
        print(f"{args.config} {name}: {ms * 1e3:8.1f} us  {nbytes / ms / 1e6:7.0f} GB/s  ({_cabi.last_path()})")


if __name__ == "__main__":
    main()
