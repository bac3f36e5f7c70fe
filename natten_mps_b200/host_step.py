"""Fused forward + backward for tensors that live in (pinned) host memory.

A training step whose activations arrive from the host pays for the PCIe copies in both
directions.  ``HostStep`` cuts the batch into slices and runs three CUDA streams so that slice
``i`` computes while slice ``i+1`` is copied in and the gradients of slice ``i-1`` are copied
out; both copy directions are busy at once.  The arithmetic is exactly the fused operator's
(``na{1,2,3}d`` forward, then its backward for a given ``dout``): the batch axis is independent,
so slicing changes no result bit.

    step = HostStep(rank=2, kernel_size=7)
    out_h, dq_h, dk_h, dv_h = step(q_h, k_h, v_h, dout_h)      # pinned host tensors in and out
    step.synchronize()                                         # results are ready after this

There is no counterpart in the reference (``src/natten_mps/functional.py`` works on tensors of one
device); the semantics of the two calls it fuses are those of ``na*d`` (functional.py:243-322) and
of the autograd backward (autograd/_factory.py:63-102).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _cabi
from .utils.params import (check_dilation_kernel_vs_input, check_kernel_size_vs_input,
                           check_stride_vs_kernel, normalize_kernel_size, normalize_tuple_param)


class HostStep:
    def __init__(self, rank: int, kernel_size, stride=1, dilation=1, is_causal=False,
                 scale: Optional[float] = None, slices: int = 4, device=None, want_out: bool = False):
        if rank not in (1, 2, 3):
            raise ValueError("rank must be 1, 2 or 3.")
        if slices < 1:
            raise ValueError("slices must be >= 1.")
        self.rank = rank
        self.ks = normalize_kernel_size(kernel_size, rank)
        self.st = normalize_tuple_param(stride, rank, "stride")
        self.dil = normalize_tuple_param(dilation, rank, "dilation")
        causal = normalize_tuple_param(is_causal, rank, "is_causal")
        if not all(isinstance(c, bool) for c in causal):
            raise ValueError("is_causal must be a bool or a tuple of bools.")
        self.causal = causal
        check_stride_vs_kernel(self.st, self.ks)
        self.scale = scale
        self.slices = slices
        self.want_out = want_out
        if not torch.cuda.is_available():
            raise RuntimeError("HostStep needs a CUDA device (there is no CPU path).")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._s_in = torch.cuda.Stream(self.device)
        self._s_cmp = torch.cuda.Stream(self.device)
        self._s_out = torch.cuda.Stream(self.device)
        self._stage = None           # device staging buffers, kept between calls
        self._host = None            # pinned result buffers, kept between calls
        self._key = None
        self._free = []              # per slice: event after which its staging buffers may be overwritten
        self._copied = []            # per slice: event after which its device results may be overwritten

    # -- buffers ------------------------------------------------------------------------
    def _bounds(self, batch: int):
        n = min(self.slices, batch)
        base, rem = divmod(batch, n)
        edges = [0]
        for i in range(n):
            edges.append(edges[-1] + base + (1 if i < rem else 0))
        return [(edges[i], edges[i + 1]) for i in range(n)]

    def _prepare(self, q, k, v):
        key = (tuple(q.shape), tuple(k.shape), tuple(v.shape), q.dtype)
        if key == self._key:
            return
        # The old buffers were used on the side streams: nothing queued there may still touch them
        # when the allocator gets them back.
        self._drain()
        dev = self.device
        rank = self.rank
        osp = tuple(-(-n // s) for n, s in zip(q.shape[1:1 + rank], self.st))
        out_shape = (q.shape[0], *osp, q.shape[-2], v.shape[-1])
        with torch.cuda.device(dev):
            # inputs (q, k, v, dout) and every result live in buffers that are allocated once:
            # the step itself never touches the allocator
            self._stage = [torch.empty(t.shape, dtype=t.dtype, device=dev) for t in (q, k, v)]
            self._stage.append(torch.empty(out_shape, dtype=q.dtype, device=dev))          # dout
            acc = torch.float64 if q.dtype == torch.float64 else torch.float32
            self._dev_out = torch.empty(out_shape, dtype=q.dtype, device=dev)
            self._dev_lse = torch.empty(out_shape[:-1], dtype=acc, device=dev)
            self._dev_grads = [torch.empty(t.shape, dtype=t.dtype, device=dev) for t in (q, k, v)]
        shapes = [out_shape, q.shape, k.shape, v.shape]
        self._host = [torch.empty(s, dtype=q.dtype).pin_memory() for s in shapes]
        # one parameter block per slice (slices differ in batch size only), one workspace for all
        lib = _cabi.lib()
        scale = q.shape[-1] ** -0.5 if self.scale is None else float(self.scale)
        self._params = []
        ws_bytes = 256
        for lo, hi in self._bounds(q.shape[0]):
            qs, ks_, vs = (_cabi.token_strides(t[lo:hi], rank) for t in self._stage[:3])
            prm = _cabi.make_params(rank, q.dtype, hi - lo, q.shape[-2], k.shape[-2], q.shape[-1], v.shape[-1],
                                    q.shape[1:1 + rank], self.ks, self.st, self.dil, self.causal, scale, 0,
                                    qs, ks_, vs)
            self._params.append(prm)
            ws_bytes = max(ws_bytes, int(lib.natten_workspace_bytes(prm, _cabi.OP_FUSED_BWD)))
        self._ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        self._key = key

    def _drain(self):
        for st in (self._s_in, self._s_cmp, self._s_out):
            st.synchronize()
        self._free, self._copied = [], []

    def close(self):
        """Wait for queued work and release the device and pinned buffers."""
        self._drain()
        self._stage = self._host = self._key = None
        self._dev_out = self._dev_lse = self._dev_grads = self._ws = None

    def __del__(self):
        try:
            self._drain()
        except Exception:      # interpreter shutdown: the context may already be gone
            pass

    # -- the step -----------------------------------------------------------------------
    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dout: torch.Tensor):
        """-> (out or None, dq, dk, dv): pinned host tensors owned by this object (overwritten by the
        next call).  The work is only queued: call ``synchronize()`` (or ``wait()`` and then synchronise
        the current stream) before reading them.  Successive calls overlap: the next call's copies in
        run while this call's gradients are still on their way out."""
        for name, t in (("query", q), ("key", k), ("value", v), ("dout", dout)):
            if t.device.type != "cpu":
                raise ValueError(f"{name} must be a host tensor.")
            if t.ndim != self.rank + 3:
                raise ValueError(f"{name} must have {self.rank + 3} dimensions.")
            if t.dtype != q.dtype:
                raise ValueError("query, key, value and dout must share one dtype.")
        if k.shape != v.shape[:-1] + (k.shape[-1],) or q.shape[:-2] != k.shape[:-2]:
            raise ValueError("query, key and value must agree on batch and spatial dimensions.")
        spatial = tuple(q.shape[1:1 + self.rank])
        check_kernel_size_vs_input(self.ks, spatial)
        check_dilation_kernel_vs_input(self.dil, self.ks, spatial)
        self._prepare(q, k, v)
        if tuple(dout.shape) != tuple(self._stage[3].shape):
            raise ValueError(f"dout must have shape {tuple(self._stage[3].shape)}.")

        cur = torch.cuda.current_stream(self.device)
        self._s_in.wait_stream(cur)            # after whatever the caller queued
        bounds = self._bounds(q.shape[0])
        if len(self._free) != len(bounds):
            self._free = [None] * len(bounds)
            self._copied = [None] * len(bounds)
        srcs = (q, k, v, dout)
        for i, (lo, hi) in enumerate(bounds):
            with torch.cuda.stream(self._s_in):
                if self._free[i] is not None:  # the previous call has finished with this staging slice
                    self._s_in.wait_event(self._free[i])
                for dst, src in zip(self._stage, srcs):
                    dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self._s_in)
            with torch.cuda.stream(self._s_cmp):
                self._s_cmp.wait_event(ready)
                if self._copied[i] is not None:   # the previous call's results of this slice are on the host
                    self._s_cmp.wait_event(self._copied[i])
                self._launch(i, lo, hi)
                done = torch.cuda.Event()
                done.record(self._s_cmp)
                self._free[i] = done
            with torch.cuda.stream(self._s_out):
                self._s_out.wait_event(done)
                results = (self._dev_out if self.want_out else None, *self._dev_grads)
                for dst, src in zip(self._host, results):
                    if src is not None:
                        dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
                copied = torch.cuda.Event()
                copied.record(self._s_out)
                self._copied[i] = copied
        return (self._host[0] if self.want_out else None, self._host[1], self._host[2], self._host[3])

    def _launch(self, i: int, lo: int, hi: int) -> None:
        """Forward + backward of batch slice [lo, hi) on the current (compute) stream, through the C ABI."""
        lib = _cabi.lib()
        prm = self._params[i]
        q, k, v, go = (t[lo:hi] for t in self._stage)
        out, lse = self._dev_out[lo:hi], self._dev_lse[lo:hi]
        dq, dk, dv = (t[lo:hi] for t in self._dev_grads)
        stream = _cabi.stream_of(q)
        with torch.cuda.device(self.device):
            rc = lib.natten_fused_fwd(prm, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), None, None, _cabi.ptr(out),
                                      _cabi.ptr(lse), stream)
            _cabi.check(rc, "natten_fused_fwd")
            rc = lib.natten_fused_bwd(prm, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), None, None, _cabi.ptr(out),
                                      _cabi.ptr(lse), _cabi.ptr(go), None, _cabi.ptr(dq), _cabi.ptr(dk), _cabi.ptr(dv),
                                      None, None, _cabi.ptr(self._ws), self._ws.numel(), stream)
            _cabi.check(rc, "natten_fused_bwd")
        if i == len(self._params) - 1:         # once per step: status word -> pinned host word
            _cabi.track_status(q)

    def wait(self):
        """Make the caller's current stream wait for everything queued so far (the copies out included)."""
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self._s_out)
        cur.wait_stream(self._s_cmp)

    def synchronize(self):
        """Block the host until the results of every call so far are in host memory; raises if a
        kernel reported a timed-out wait."""
        self._s_out.synchronize()
        self._s_cmp.synchronize()
        _cabi.poll_status(self.device)

    # -- traffic, for reports -----------------------------------------------------------
    def bytes_per_step(self, q, k, v, dout):
        h2d = sum(t.numel() * t.element_size() for t in (q, k, v, dout))
        d2h = sum(t.numel() * t.element_size() for t in (q, k, v)) + (dout.numel() * dout.element_size() if self.want_out else 0)
        return h2d, d2h
