#!/usr/bin/env python
"""Benchmark of the neighbourhood-attention hot path (fused forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2]

One "step" is one forward + one backward of the workload through the C ABI
(``natten_fused_fwd`` + ``natten_fused_bwd``) on tensors already resident in HBM.
Prints ONE JSON line (rank 0).  With N > 1 (launched by torchrun, one rank per
GPU) every rank runs the same per-GPU workload on its own shard of the global
batch -- the path has no exchange step, so there is no collective in the timed
region; NCCL only carries the barrier and the max-over-ranks of the timings.

Beside the headline (weak scaling, per-GPU batch fixed) the line carries
  * ``other_configs``   the other benchmark configurations (1-GPU runs only), timed in the same process;
  * ``split_ops``       the split QK / AV operators at the headline shape (1-GPU runs only);
  * ``strong_scaling``  the headline configuration and the ragged long-sequence configuration at FIXED
                        global size, cut across the ranks by ``natten_mps_b200.sharding``;
  * ``e2e``             the same step through ``HostStep`` with host buffers, and a copy-only control
                        that moves the same bytes without any kernel.

``--impl reference`` times the CPU restatement of the reference's pure backend
(``oracle/``) on the host cores, on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c1": dict(rank=1, B=2, spatial=(128,), Hq=4, Hkv=4, D=32, kernel=(7,), dilation=(1,),
               stride=(1,), causal=(False,), dtype="f32", bound="latency",
               desc="na1d fp32 fwd+bwd B=2 L=128 heads=4 head_dim=32 kernel=7"),
    "c2": dict(rank=2, B=8, spatial=(64, 64), Hq=8, Hkv=8, D=64, kernel=(7, 7), dilation=(1, 1),
               stride=(1, 1), causal=(False, False), dtype="bf16", bound="hbm",
               desc="na2d bf16 fwd+bwd B=8 64x64 heads=8 head_dim=64 kernel=7x7"),
    "c3": dict(rank=2, B=4, spatial=(128, 128), Hq=8, Hkv=8, D=64, kernel=(13, 13), dilation=(2, 2),
               stride=(1, 1), causal=(False, False), dtype="bf16", bound="hbm",
               desc="na2d bf16 fwd+bwd B=4 128x128 heads=8 head_dim=64 kernel=13x13 dilation=2"),
    "c3s": dict(rank=2, B=4, spatial=(128, 128), Hq=8, Hkv=8, D=64, kernel=(13, 13), dilation=(2, 2),
                stride=(2, 2), causal=(False, False), dtype="bf16", bound="hbm", forward_only=True,
                desc="na2d bf16 forward B=4 128x128 heads=8 head_dim=64 kernel=13x13 dilation=2 stride=2"),
    "c4": dict(rank=3, B=2, spatial=(16, 32, 32), Hq=8, Hkv=8, D=64, kernel=(3, 7, 7),
               dilation=(1, 1, 1), stride=(1, 1, 1), causal=(True, False, False), dtype="bf16", bound="hbm",
               desc="na3d bf16 fwd+bwd B=2 16x32x32 heads=8 head_dim=64 kernel=3x7x7 causal-D"),
    "c5": dict(rank=1, B=8, spatial=(16384,), Hq=16, Hkv=4, D=128, kernel=(255,), dilation=(1,),
               stride=(1,), causal=(False,), dtype="f16", bound="tensor", n_extra=16, varlen=(4096, 16385),
               desc="na1d fp16 fwd+bwd B=8 L<=16384 (valid lengths uniform in [4096,16384]) heads=16/4 "
                    "head_dim=128 kernel=255 + 16 additional tokens"),
}
ESIZE = {"bf16": 2, "f16": 2, "f32": 4}


def mean_valid_keys(w) -> float:
    """Average number of unmasked keys per query (only causal axes mask anything)."""
    k_eff = 1.0
    for L, K, dil, causal in zip(w["spatial"], w["kernel"], w["dilation"], w["causal"]):
        if causal:
            k_eff *= sum(min(K, p // dil + 1) for p in range(L)) / L
        else:
            k_eff *= K
    return k_eff + w.get("n_extra", 0)


def algorithmic(w, batch, lens=None):
    """(flops fwd, flops fwd+bwd, bytes fwd, bytes bwd) of one step.  4*N_qh*K_eff*D flops forward,
    12* forward+backward (the recomputed scores are not counted); every tensor touched once at its
    storage width, lse float32.  ``lens``: valid tokens per sample (ragged workload)."""
    if lens is not None:
        n_in = n_out = float(sum(lens))
    else:
        n_in, n_out = float(batch), float(batch)
        for s, st in zip(w["spatial"], w["stride"]):
            n_in *= s
            n_out *= -(-s // st)
    esz = ESIZE[w["dtype"]]
    n_qh = n_out * w["Hq"]
    fwd_flops = 4.0 * n_qh * mean_valid_keys(w) * w["D"]
    q_in = n_in * w["Hq"] * w["D"] * esz
    q_out = n_out * w["Hq"] * w["D"] * esz
    kv = n_in * w["Hkv"] * w["D"] * esz
    lse = n_qh * 4
    fwd = q_in + q_out + 2 * kv + lse                                # q, o, k, v, lse
    bwd = 2 * q_in + 2 * q_out + 4 * kv + lse                        # q, dq, o, do, k, v, dk, dv, lse
    return fwd_flops, 3.0 * fwd_flops, fwd, bwd


class ClockSampler:
    """Samples SM clocks and throttle reasons every 100 ms with one streaming nvidia-smi
    process for as long as the timed sections run."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._proc, self._t = index, [], None, None

    def _pump(self):
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.strip().split(",")]
            if len(parts) >= 6:
                self.rows.append(parts)

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._pump, daemon=True)
            self._t.start()
        except Exception:
            self._proc = None
        return self

    def __exit__(self, *exc):
        if self._proc is not None:
            self._proc.terminate()          # the exact process started above
            try:
                self._proc.wait(timeout=5)
            except Exception:
                self._proc.kill()
            self._t.join(timeout=5)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        num = lambda x: x.replace(".", "", 1).isdigit()
        sm = [float(r[0]) for r in self.rows if num(r[0])]
        mx = [float(r[1]) for r in self.rows if num(r[1])]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def ncu_traffic(workload, phase, batch):
    """DRAM bytes (read + write) per launch set from the last profiler capture, scaled to `batch`
    (the traffic grows in proportion to the batch).  The capture's numbers live in a small data
    file next to the profile summaries; None when there is no capture for this workload."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f)[workload]
        return float(rec[phase]) * batch / float(rec["batch"])
    except Exception:
        return None


def config_of(w, batch, world, lens=None):
    """The keys both arms report, so that their lines describe the same configuration."""
    fwd_flops, flops, fwd_bytes, bwd_bytes = algorithmic(w, batch, lens)
    return {"workload": w["desc"], "per_gpu_batch": batch, "global_batch": batch * world,
            "sharding": "batch, no collective",
            "algorithmic_gflop_per_step": flops / 1e9,
            "algorithmic_gb_per_step": (fwd_bytes + bwd_bytes) / 1e9}


# ---------------------------------------------------------------------------
# CPU arms
# ---------------------------------------------------------------------------
def cpu_port_run(w, steps, warmup, sample_batch):
    """The C restatement of the reference's pure backend (oracle/), OpenMP over the host cores."""
    import numpy as np
    import oracle
    rng = np.random.default_rng(0)
    shp_q = (sample_batch, *w["spatial"], w["Hq"], w["D"])
    shp_k = (sample_batch, *w["spatial"], w["Hkv"], w["D"])
    q = rng.standard_normal(shp_q, dtype=np.float32)
    k = rng.standard_normal(shp_k, dtype=np.float32)
    v = rng.standard_normal(shp_k, dtype=np.float32)
    go = rng.standard_normal(shp_q, dtype=np.float32)
    kw = dict(kernel_size=w["kernel"], stride=w["stride"], dilation=w["dilation"], is_causal=w["causal"],
              dtype=np.float32)

    def step():
        out, lse = oracle.na_forward(q, k, v, **kw)
        oracle.na_backward(q, k, v, out, lse, go, **kw)

    for _ in range(warmup):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    _, flops, _, _ = algorithmic(w, sample_batch)
    sec = sum(times) / len(times)
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"batch {sample_batch} of {w['B']} of the workload, float32, OpenMP over all host "
                      f"cores, mean of {steps} step(s), {sec * 1e3:.1f} ms/step"}, sec


def cpu_pure_run(w, sample_batch=1):
    """The reference's own pure-PyTorch backend (``functional.na*d`` + autograd, float32) when the
    reference package has been installed next to this file (``baseline/_ref``); a bounded sample."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "natten_mps")):
        return "unavailable on this box"
    try:
        import torch
        os.environ["NATTEN_BACKEND"] = "pure"
        sys.path.insert(0, ref)
        from natten_mps import functional as RF
        fn = {1: RF.na1d, 2: RF.na2d, 3: RF.na3d}[w["rank"]]
        torch.set_num_threads(os.cpu_count())
        g = torch.Generator().manual_seed(0)
        mk = lambda h: torch.randn((sample_batch, *w["spatial"], h, w["D"]), generator=g)
        q, k, v, go = mk(w["Hq"]), mk(w["Hkv"]), mk(w["Hkv"]), mk(w["Hq"])
        times = []
        for i in range(3):                       # one warm-up, two timed
            leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
            t0 = time.perf_counter()
            out = fn(*leaves, kernel_size=w["kernel"], stride=w["stride"], dilation=w["dilation"],
                     is_causal=w["causal"])
            out.backward(go)
            if i:
                times.append(time.perf_counter() - t0)
        sec = sum(times) / len(times)
        _, flops, _, _ = algorithmic(w, sample_batch)
        return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "reference",
                "sample": f"batch {sample_batch} of {w['B']} of the workload, float32, the reference's pure backend "
                          f"through functional.na{w['rank']}d + autograd, mean of 2 steps, {sec * 1e3:.0f} ms/step"}
    except Exception as exc:                      # the baseline is a report, never a reason to fail
        return f"unavailable on this box ({type(exc).__name__}: {exc})"
    finally:
        if ref in sys.path:
            sys.path.remove(ref)


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())
    steps = max(1, min(args.steps, 20))
    warmup = max(0, min(args.warmup, 5))
    cb, sec = cpu_port_run(w, steps, warmup, sample_batch=w["B"])
    line = {
        "impl": "reference", "metric": f"na{w['rank']}d fwd+bwd TFLOP/s", "value": cb["value"],
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_of(w, w["B"], int(os.environ.get("WORLD_SIZE", "1"))),
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class Problem:
    """One workload resident on a device: tensors, parameter block and the two C-ABI calls."""

    def __init__(self, w, batch, dev, seed, pinned_host=False, lens=None):
        import ctypes
        import torch
        from natten_mps_b200 import _cabi
        self.w, self.B, self.dev = w, batch, dev
        tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[w["dtype"]]
        self.tdt = tdt
        g = torch.Generator(device="cpu").manual_seed(seed)
        osp = tuple(-(-s // st) for s, st in zip(w["spatial"], w["stride"]))
        self.shp_q = (batch, *w["spatial"], w["Hq"], w["D"])
        self.shp_k = (batch, *w["spatial"], w["Hkv"], w["D"])
        self.shp_o = (batch, *osp, w["Hq"], w["D"])
        # draw order of the benchmark recipe: q, k, v, grad_out, additional keys / values, lengths
        host = [torch.randn(s, generator=g).to(tdt) for s in (self.shp_q, self.shp_k, self.shp_k, self.shp_o)]
        ne = w.get("n_extra", 0)
        ek = ev = None
        if ne:
            ek = torch.randn((batch, ne, w["Hkv"], w["D"]), generator=g).to(tdt)
            ev = torch.randn((batch, ne, w["Hkv"], w["D"]), generator=g).to(tdt)
        self.lens = None
        ext = None
        if w.get("varlen"):
            lo, hi = w["varlen"]
            self.lens = lens if lens is not None else torch.randint(lo, hi, (batch,), generator=g, dtype=torch.int32).tolist()
            ext = torch.tensor(self.lens, dtype=torch.int32, device=dev).reshape(batch, 1)
        if pinned_host:
            host = [t.pin_memory() for t in host]
        self.host = host
        self.q, self.k, self.v, self.go = [t.to(dev) for t in host]
        self.ek, self.ev = (None if ek is None else ek.to(dev)), (None if ev is None else ev.to(dev))
        self.ext = ext
        L = _cabi.lib()
        r = w["rank"]
        strides = lambda t: _cabi.token_strides(t, r)
        self.params = _cabi.make_params(r, tdt, batch, w["Hq"], w["Hkv"], w["D"], w["D"], w["spatial"], w["kernel"],
                                        w["stride"], w["dilation"], w["causal"], w["D"] ** -0.5, ne,
                                        strides(self.q), strides(self.k), strides(self.v), ext)
        self.out = torch.empty(self.shp_o, dtype=tdt, device=dev)
        self.lse = torch.empty(self.shp_o[:-1], dtype=torch.float32, device=dev)
        self.dq, self.dk, self.dv = torch.empty_like(self.q), torch.empty_like(self.k), torch.empty_like(self.v)
        self.dek = None if ek is None else torch.empty_like(self.ek)
        self.dev_ = None if ev is None else torch.empty_like(self.ev)
        ws_bytes = int(L.natten_workspace_bytes(self.params, _cabi.OP_FUSED_BWD))
        self.ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        fa = (self.params, P(self.q), P(self.k), P(self.v), P(self.ek), P(self.ev), P(self.out), P(self.lse), stream)
        ba = (self.params, P(self.q), P(self.k), P(self.v), P(self.ek), P(self.ev), P(self.out), P(self.lse),
              P(self.go), None, P(self.dq), P(self.dk), P(self.dv), P(self.dek), P(self.dev_), P(self.ws),
              self.ws.numel(), stream)
        self.forward_only = bool(w.get("forward_only"))

        def fwd():
            rc = L.natten_fused_fwd(*fa)
            if rc:
                _cabi.check(rc, "natten_fused_fwd")

        def bwd():
            if self.forward_only:
                return
            rc = L.natten_fused_bwd(*ba)
            if rc:
                _cabi.check(rc, "natten_fused_bwd")

        self.fwd, self.bwd = fwd, bwd

    def step(self):
        self.fwd()
        self.bwd()

    def phase_times(self, reps):
        """Median forward / backward time (ms) over `reps` steps, each phase between its own events."""
        import torch
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        f, b = [], []
        for _ in range(reps):
            ev[0].record(); self.fwd(); ev[1].record(); self.bwd(); ev[2].record()
            torch.cuda.synchronize()
            f.append(ev[0].elapsed_time(ev[1])); b.append(ev[1].elapsed_time(ev[2]))
        return statistics.median(f), statistics.median(b)

    def algorithmic(self):
        return algorithmic(self.w, self.B, self.lens)


def roofline_ms(w, fwd_flops, flops, fwd_bytes, bwd_bytes, hbm_peak, tc_peak):
    """Time the faster of the two limits allows for forward and for the whole step (ms)."""
    t_f = max(fwd_bytes / (hbm_peak * 1e9), fwd_flops / (tc_peak * 1e12))
    t_s = max((fwd_bytes + bwd_bytes) / (hbm_peak * 1e9), flops / (tc_peak * 1e12))
    return t_f * 1e3, t_s * 1e3


def time_other_configs(dev, hbm_peak, tc_peak):
    import torch
    from natten_mps_b200 import _cabi
    rows = []
    for name in ("c1", "c3", "c3s", "c4", "c5"):
        w = WORKLOADS[name]
        try:
            pb = Problem(w, w["B"], dev, seed=0)
            for _ in range(3):
                pb.step()
            torch.cuda.synchronize()
            f_ms, b_ms = pb.phase_times(5)
            path = _cabi.last_path()
            fwd_flops, flops, fb, bb = pb.algorithmic()
            if pb.forward_only:
                flops, bb, b_ms = fwd_flops, 0.0, 0.0
            t_f, t_s = roofline_ms(w, fwd_flops, flops, fb, bb, hbm_peak, tc_peak)
            row = {"config": name, "workload": w["desc"], "fwd_ms": f_ms, "bwd_ms": b_ms,
                   "tflops": flops / ((f_ms + b_ms) * 1e-3) / 1e12, "bound": w["bound"],
                   "roofline_ms": t_s, "roofline_frac": (t_s / (f_ms + b_ms)) if w["bound"] != "latency" else None,
                   "kernel_path": path}
            if pb.lens is not None:
                row["valid_tokens"] = int(sum(pb.lens))
            rows.append(row)
            del pb
            torch.cuda.empty_cache()
        except Exception as exc:
            rows.append({"config": name, "error": f"{type(exc).__name__}: {exc}"})
    return rows


def time_split_ops(w, dev, hbm_peak):
    """Split QK / AV operators at the workload's shape: ms and fraction of the HBM roofline (their
    traffic is dominated by the [.., prod(kernel)]-wide logits tensor)."""
    import torch
    from natten_mps_b200 import _backend, _cabi
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[w["dtype"]]
    g = torch.Generator(device="cpu").manual_seed(5)
    B = w["B"]
    ktot = 1
    for kk in w["kernel"]:
        ktot *= kk
    q = torch.randn((B, *w["spatial"], w["Hq"], w["D"]), generator=g).to(tdt).to(dev)
    k = torch.randn((B, *w["spatial"], w["Hkv"], w["D"]), generator=g).to(tdt).to(dev)
    attn = torch.softmax(torch.randn((B, *w["spatial"], w["Hq"], ktot), generator=g), -1).to(tdt).to(dev)
    geo = (w["kernel"], w["dilation"], w["stride"], w["causal"])
    esz = ESIZE[w["dtype"]]
    qb, lb = q.numel() * esz, attn.numel() * esz
    ops = {
        "qk_fwd": (lambda: _backend.qk_forward(q, k, *geo, w["D"] ** -0.5), 2 * qb + lb),
        "av_fwd": (lambda: _backend.av_forward(attn, k, *geo), 2 * qb + lb),
        "qk_bwd": (lambda: _backend.qk_backward(attn, q, k, *geo, w["D"] ** -0.5), 4 * qb + lb),
        "av_bwd": (lambda: _backend.av_backward(q, attn, k, *geo), 3 * qb + 2 * lb),
    }
    out = {}
    for name, (fn, nbytes) in ops.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        out[name] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm_peak,
                     "kernel_path": _cabi.last_path()}
    return out


def run_ours(args, w):
    import torch
    from natten_mps_b200 import _cabi, functional as F, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the library has no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    B = w["B"]                                       # per-GPU batch (weak scaling)
    pb = Problem(w, B, dev, seed=1000 + rank, pinned_host=True)
    tdt, host = pb.tdt, pb.host
    step = pb.step

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def reduce_max(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    sync_all()

    # ---- device-resident timing: K steps between two events ------------------
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = _cabi.launch_count()
    clocks = ClockSampler(local)
    clocks.__enter__()
    time.sleep(0.25)                                  # let the sampler take its first reading
    sync_all()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync_all()
    launches = _cabi.launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    path = _cabi.last_path()

    if args.kernels_only:
        clocks.__exit__(None, None, None)
        if rank == 0:
            print(json.dumps({"ms_per_step": ms_total / args.steps, "kernel_path": path,
                              "gpu_launches": launches}), flush=True)
        return

    fwd_t, bwd_t = pb.phase_times(max(5, min(args.steps, 20)))

    # ---- end to end through the public API with host buffers -----------------
    # (a) HostStep: the package's call for host-resident tensors (batch slices over three
    #     streams, so both PCIe directions and the kernels overlap); (b) the plain autograd
    #     call on one stream; (c) a control that only moves the same bytes in and out.
    from natten_mps_b200.host_step import HostStep
    fn = {1: F.na1d, 2: F.na2d, 3: F.na3d}[w["rank"]]
    res_host = [torch.empty(s, dtype=tdt).pin_memory() for s in (pb.shp_q, pb.shp_k, pb.shp_k)]
    # every rank copies through the same host: fewer, larger copies when many ranks share it
    slices = min(8 if world < 4 else 2, B)
    host_step = HostStep(w["rank"], w["kernel"], stride=w["stride"], dilation=w["dilation"],
                         is_causal=w["causal"], slices=slices, device=dev)
    copy_streams = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
    dev_in = [pb.q, pb.k, pb.v, pb.go]
    dev_res = [pb.dq, pb.dk, pb.dv]

    def e2e_step():
        host_step(*host)          # successive steps overlap, as a data pipeline would run them

    def e2e_latency_step():
        host_step(*host)
        host_step.synchronize()   # one isolated step, nothing overlapped with its neighbours

    def e2e_autograd_step():
        qd, kd, vd, gd = [t.to(dev, non_blocking=True) for t in host]
        qd.requires_grad_(True); kd.requires_grad_(True); vd.requires_grad_(True)
        o = fn(qd, kd, vd, kernel_size=w["kernel"], stride=w["stride"], dilation=w["dilation"],
               is_causal=w["causal"])
        o.backward(gd)
        for dst, src in zip(res_host, (qd.grad, kd.grad, vd.grad)):
            dst.copy_(src, non_blocking=True)

    def copy_only_step():         # the same bytes in and out on two streams, no kernel at all
        with torch.cuda.stream(copy_streams[0]):
            for d, s in zip(dev_in, host):
                d.copy_(s, non_blocking=True)
        with torch.cuda.stream(copy_streams[1]):
            for d, s in zip(res_host, dev_res):
                d.copy_(s, non_blocking=True)

    def time_e2e(fn_step):
        for _ in range(3):
            fn_step()
        host_step.wait()
        for cs in copy_streams:
            torch.cuda.current_stream(dev).wait_stream(cs)
        sync_all()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = max(3, min(args.steps, 10))
        e2.record()
        for _ in range(n):
            fn_step()
        host_step.wait()          # the closing event sits on the current stream: it must see the side streams
        for cs in copy_streams:
            torch.cuda.current_stream(dev).wait_stream(cs)
        e3.record()
        sync_all()
        return e2.elapsed_time(e3) / n

    e2e_ms = time_e2e(e2e_step)
    e2e_autograd_ms = time_e2e(e2e_autograd_step)
    e2e_latency_ms = time_e2e(e2e_latency_step)
    copy_only_ms = time_e2e(copy_only_step)

    # ---- strong scaling: fixed global problems cut across the ranks ----------
    strong = {}
    try:
        # (a) the headline configuration, global batch = w["B"], contiguous batch slices
        sl = sharding.batch_slice(w["B"], rank, world)
        nb = sl.stop - sl.start
        if nb > 0:
            ps = Problem(w, nb, dev, seed=2000 + rank)
            for _ in range(3):
                ps.step()
        sync_all()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_strong = max(5, min(args.steps, 50))
        s0.record()
        if nb > 0:
            for _ in range(n_strong):
                ps.step()
        s1.record()
        sync_all()
        t_fixed = reduce_max([s0.elapsed_time(s1) / n_strong])[0]
        _, flops_fixed, _, _ = algorithmic(w, w["B"])
        strong["fixed_global_batch"] = {"workload": w["desc"], "global_batch": w["B"], "per_rank_batch": nb,
                                        "split": "sharding.batch_slice", "ms_per_step": t_fixed,
                                        "tflops": flops_fixed / (t_fixed * 1e-3) / 1e12}
        if nb > 0:
            del ps
        # (b) the ragged long-sequence configuration: samples assigned longest-first by valid length
        w5 = WORKLOADS["c5"]
        g5 = torch.Generator(device="cpu").manual_seed(0)
        lens_all = torch.randint(w5["varlen"][0], w5["varlen"][1], (w5["B"],), generator=g5, dtype=torch.int32).tolist()
        mine = sharding.assign_units(lens_all, world)[rank]
        if mine:
            p5 = Problem(w5, len(mine), dev, seed=3000 + rank, lens=[lens_all[i] for i in mine])
            for _ in range(2):
                p5.step()
        sync_all()
        s0.record()
        if mine:
            for _ in range(3):
                p5.step()
        s1.record()
        sync_all()
        t5 = reduce_max([s0.elapsed_time(s1) / 3])[0]
        _, flops5, _, _ = algorithmic(w5, w5["B"], lens_all)
        strong["ragged_long_sequences"] = {"workload": w5["desc"], "samples": w5["B"], "samples_of_rank0": len(mine),
                                           "split": "sharding.assign_units by valid length", "ms_per_step": t5,
                                           "tflops": flops5 / (t5 * 1e-3) / 1e12}
        if mine:
            del p5
        torch.cuda.empty_cache()
    except Exception as exc:
        strong["error"] = f"{type(exc).__name__}: {exc}"

    # keep the GPU busy a little longer so that the clock record has samples under load
    t_end = time.time() + 0.6
    while time.time() < t_end:
        for _ in range(20):
            step()
        torch.cuda.synchronize()
    clocks.__exit__(None, None, None)

    # ---- reduce over ranks ---------------------------------------------------
    ms_total, e2e_ms, fwd_t, bwd_t, e2e_autograd_ms, e2e_latency_ms, copy_only_ms = reduce_max(
        [ms_total, e2e_ms, fwd_t, bwd_t, e2e_autograd_ms, e2e_latency_ms, copy_only_ms])
    ms_step = ms_total / args.steps
    fwd_flops, flops, fwd_bytes, bwd_bytes = pb.algorithmic()
    hbm_peak, tc_peak, which = measured_peaks()
    dominant = ("backward", bwd_t, bwd_bytes) if bwd_t >= fwd_t else ("forward", fwd_t, fwd_bytes)
    achieved = dominant[2] / (dominant[1] * 1e-3) / 1e9
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = sum(t.numel() * t.element_size() for t in res_host)

    if rank == 0:
        line = {
            "metric": f"na{w['rank']}d fwd+bwd TFLOP/s", "value": world * flops / (ms_step * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": w["dtype"], "data": "synthetic",
            "config": config_of(w, B, world),
            "kernel_path": path,
            "l2": "working set per step (0.40 GB at c2) exceeds the 126 MB L2; no explicit flush",
            "fwd_ms": fwd_t, "bwd_ms": bwd_t,
            "roofline": {"bound": "hbm", "kernel": dominant[0], "achieved": achieved, "peak": hbm_peak,
                         "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": ncu_traffic(args.workload, dominant[0], B),
                         "peak_source": which,
                         "step_frac": ((fwd_bytes + bwd_bytes) / (ms_step * 1e-3) / 1e9) / hbm_peak,
                         "step_frac_nominal_8tbs": ((fwd_bytes + bwd_bytes) / (ms_step * 1e-3) / 1e9) / 8000.0},
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": f"natten_mps_b200.HostStep ({slices} batch slices over copy-in / compute / copy-out streams)",
                    "isolated_step_ms": e2e_latency_ms, "autograd_api_ms_per_step": e2e_autograd_ms,
                    "copy_only_ms_per_step": copy_only_ms,
                    "frac_of_copy_ceiling": copy_only_ms / e2e_ms if e2e_ms > 0 else None},
            "strong_scaling": strong,
            "gpu_launches": launches,
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_extras:
            line["other_configs"] = time_other_configs(dev, hbm_peak, tc_peak)
            line["split_ops"] = time_split_ops(w, dev, hbm_peak)
        if world == 1 and not args.no_cpu_baseline:
            os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())
            line["cpu_baseline"], _ = cpu_port_run(w, steps=5, warmup=1, sample_batch=w["B"])
            line["cpu_baseline_pure"] = cpu_pure_run(w, sample_batch=min(2, w["B"]))
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip other_configs / split_ops")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the per-GPU batch (small cases for profiler captures)")
    ap.add_argument("--kernels-only", action="store_true",
                    help="only the device-resident timed loop (for profiler captures)")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.batch > 0:
        w["B"] = args.batch
        w["desc"] += f" (batch overridden to {args.batch})"
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
