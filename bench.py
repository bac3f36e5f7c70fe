#!/usr/bin/env python
"""Benchmark of the neighbourhood-attention hot path (fused forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2]

One "step" is one forward + one backward of the workload through the C ABI
(``natten_fused_fwd`` + ``natten_fused_bwd``) on tensors already resident in HBM.
Prints ONE JSON line (rank 0).  With N > 1 (launched by torchrun, one rank per
GPU) every rank runs the same per-GPU workload on its own shard of the global
batch -- the path has no exchange step, so there is no collective in the timed
region; NCCL only carries the barrier and the max-over-ranks of the timings.

``--impl reference`` times the CPU restatement of the reference's pure backend
(``oracle/``) on the host cores, on a bounded sample of the same workload.
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

# name -> (rank, B, spatial, Hq, Hkv, D, kernel, dilation, stride, causal, dtype)
WORKLOADS = {
    "c2": dict(rank=2, B=8, spatial=(64, 64), Hq=8, Hkv=8, D=64, kernel=(7, 7), dilation=(1, 1),
               stride=(1, 1), causal=(False, False), dtype="bf16",
               desc="na2d bf16 fwd+bwd B=8 64x64 heads=8 head_dim=64 kernel=7x7"),
    "c3": dict(rank=2, B=4, spatial=(128, 128), Hq=8, Hkv=8, D=64, kernel=(13, 13), dilation=(2, 2),
               stride=(1, 1), causal=(False, False), dtype="bf16",
               desc="na2d bf16 fwd+bwd B=4 128x128 heads=8 head_dim=64 kernel=13x13 dilation=2"),
    "c4": dict(rank=3, B=2, spatial=(16, 32, 32), Hq=8, Hkv=8, D=64, kernel=(3, 7, 7),
               dilation=(1, 1, 1), stride=(1, 1, 1), causal=(True, False, False), dtype="bf16",
               desc="na3d bf16 fwd+bwd B=2 16x32x32 heads=8 head_dim=64 kernel=3x7x7 causal-D"),
    "c1": dict(rank=1, B=2, spatial=(128,), Hq=4, Hkv=4, D=32, kernel=(7,), dilation=(1,),
               stride=(1,), causal=(False,), dtype="f32",
               desc="na1d fp32 fwd+bwd B=2 L=128 heads=4 head_dim=32 kernel=7"),
}


def mean_valid_keys(w) -> float:
    """Average number of unmasked keys per query (only causal axes mask anything)."""
    k_eff = 1.0
    for L, K, dil, causal in zip(w["spatial"], w["kernel"], w["dilation"], w["causal"]):
        if causal:
            k_eff *= sum(min(K, p // dil + 1) for p in range(L)) / L
        else:
            k_eff *= K
    return k_eff


def algorithmic(w, batch):
    """(flops fwd+bwd, bytes fwd, bytes bwd) of one step: 12*N_qh*K_eff*D flops; every
    tensor touched once at its storage width, lse float32."""
    n_tok = batch
    for s in w["spatial"]:
        n_tok *= s
    esz = {"bf16": 2, "f16": 2, "f32": 4}[w["dtype"]]
    n_qh = n_tok * w["Hq"]
    flops = 12.0 * n_qh * mean_valid_keys(w) * w["D"]
    q_bytes = n_tok * w["Hq"] * w["D"] * esz
    kv_bytes = n_tok * w["Hkv"] * w["D"] * esz
    lse_bytes = n_qh * 4
    fwd = 2 * q_bytes + 2 * kv_bytes + lse_bytes                     # q, o, k, v, lse
    bwd = 4 * q_bytes + 4 * kv_bytes + lse_bytes                     # q, o, do, dq, k, v, dk, dv, lse
    return flops, fwd, bwd


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


# DRAM bytes (read + write) the backward / forward kernels move per launch set at config 2, batch 8,
# from the committed ncu capture (profiles/c2_na2d_7x7_bf16_tc_kernels_ncu_full.md); scales with batch.
NCU_TRAFFIC_C2 = {"backward": 390.2e6, "forward": 114.2e6}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


# ---------------------------------------------------------------------------
# CPU arm: the oracle (port of the reference's pure backend) on the host cores
# ---------------------------------------------------------------------------
def cpu_port_run(w, steps, warmup, sample_batch):
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
    flops, _, _ = algorithmic(w, sample_batch)
    sec = sum(times) / len(times)
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"batch {sample_batch} of {w['B']} of the workload, float32, OpenMP over all host "
                      f"cores, mean of {steps} step(s), {sec * 1e3:.1f} ms/step"}, sec


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())
    steps = max(1, min(args.steps, 20))
    cb, sec = cpu_port_run(w, steps, max(1, min(args.warmup, 2)), sample_batch=w["B"])
    line = {
        "impl": "reference", "metric": f"na{w['rank']}d fwd+bwd TFLOP/s", "value": cb["value"],
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps, "warmup": max(1, min(args.warmup, 2)),
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["desc"], "sample": cb["sample"]},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_ours(args, w):
    import torch
    from natten_mps_b200 import _backend, _cabi, functional as F

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

    tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[w["dtype"]]
    B = w["B"]                                       # per-GPU batch (weak scaling)
    g = torch.Generator(device="cpu").manual_seed(1000 + rank)
    shp_q = (B, *w["spatial"], w["Hq"], w["D"])
    shp_k = (B, *w["spatial"], w["Hkv"], w["D"])
    host = [torch.randn(s, generator=g).to(tdt).pin_memory() for s in (shp_q, shp_k, shp_k, shp_q)]
    q, k, v, go = [t.to(dev) for t in host]
    geo = dict(kernel_size=w["kernel"], stride=w["stride"], dilation=w["dilation"], is_causal=w["causal"],
               scale=w["D"] ** -0.5)

    # The timed step calls the C ABI directly on preallocated buffers (the library never
    # allocates), so the host does little more than two foreign calls per step.
    import ctypes
    L = _cabi.lib()
    rank_sp = w["rank"]
    strides = lambda t: _cabi.token_strides(t, rank_sp)
    params = _cabi.make_params(rank_sp, tdt, B, w["Hq"], w["Hkv"], w["D"], w["D"], w["spatial"], w["kernel"],
                               w["stride"], w["dilation"], w["causal"], w["D"] ** -0.5, 0,
                               strides(q), strides(k), strides(v))
    out_b = torch.empty(shp_q, dtype=tdt, device=dev)
    lse_b = torch.empty(shp_q[:-1], dtype=torch.float32, device=dev)
    dq_b, dk_b, dv_b = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws_bytes = int(L.natten_workspace_bytes(params, _cabi.OP_FUSED_BWD))
    ws_b = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    fwd_args = (params, P(q), P(k), P(v), None, None, P(out_b), P(lse_b), stream)
    bwd_args = (params, P(q), P(k), P(v), None, None, P(out_b), P(lse_b), P(go), None, P(dq_b), P(dk_b),
                P(dv_b), None, None, P(ws_b), ws_b.numel(), stream)

    def fwd_call():
        rc = L.natten_fused_fwd(*fwd_args)
        if rc:
            _cabi.check(rc, "natten_fused_fwd")

    def bwd_call():
        rc = L.natten_fused_bwd(*bwd_args)
        if rc:
            _cabi.check(rc, "natten_fused_bwd")

    def step():
        fwd_call()
        bwd_call()

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
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

    # ---- per-phase timing (forward kernel vs backward kernels) ---------------
    fe = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    fwd_ms, bwd_ms = [], []
    for _ in range(max(5, min(args.steps, 20))):
        fe[0].record()
        fwd_call()
        fe[1].record()
        bwd_call()
        fe[2].record()
        torch.cuda.synchronize()
        fwd_ms.append(fe[0].elapsed_time(fe[1]))
        bwd_ms.append(fe[1].elapsed_time(fe[2]))
    fwd_t, bwd_t = statistics.median(fwd_ms), statistics.median(bwd_ms)

    # ---- end to end through the public API with host buffers -----------------
    # (a) HostStep: the package's call for host-resident tensors (batch slices over three
    #     streams, so both PCIe directions and the kernels overlap); (b) the plain autograd
    #     call on one stream, for comparison.  Both copy every input in and every gradient out.
    from natten_mps_b200.host_step import HostStep
    fn = {1: F.na1d, 2: F.na2d, 3: F.na3d}[w["rank"]]
    res_host = [torch.empty(s, dtype=tdt).pin_memory() for s in (shp_q, shp_k, shp_k)]
    host_step = HostStep(w["rank"], w["kernel"], stride=w["stride"], dilation=w["dilation"],
                         is_causal=w["causal"], slices=min(8, B), device=dev)

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

    def time_e2e(fn_step):
        for _ in range(3):
            fn_step()
        host_step.wait()
        sync_all()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = max(3, min(args.steps, 10))
        e2.record()
        for _ in range(n):
            fn_step()
        host_step.wait()          # the closing event sits on the current stream: it must see the side streams
        e3.record()
        sync_all()
        return e2.elapsed_time(e3) / n

    e2e_ms = time_e2e(e2e_step)
    e2e_autograd_ms = time_e2e(e2e_autograd_step)
    e2e_latency_ms = time_e2e(e2e_latency_step)
    # keep the GPU busy a little longer so that the clock record has samples under load
    t_end = time.time() + 0.6
    while time.time() < t_end:
        for _ in range(20):
            step()
        torch.cuda.synchronize()
    clocks.__exit__(None, None, None)

    # ---- reduce over ranks ---------------------------------------------------
    vals = torch.tensor([ms_total, e2e_ms, fwd_t, bwd_t, e2e_autograd_ms, e2e_latency_ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, fwd_t, bwd_t, e2e_autograd_ms, e2e_latency_ms = vals.tolist()
    ms_step = ms_total / args.steps
    flops, fwd_bytes, bwd_bytes = algorithmic(w, B)
    hbm_peak, tc_peak, which = measured_peaks()
    dominant = ("backward", bwd_t, bwd_bytes) if bwd_t >= fwd_t else ("forward", fwd_t, fwd_bytes)
    achieved = dominant[2] / (dominant[1] * 1e-3) / 1e9
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = sum(t.numel() * t.element_size() for t in res_host)

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu, _ = cpu_port_run(w, steps=5, warmup=1, sample_batch=w["B"])
        line = {
            "metric": f"na{w['rank']}d fwd+bwd TFLOP/s", "value": world * flops / (ms_step * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": w["desc"], "per_gpu_batch": B, "global_batch": B * world,
                       "sharding": "batch, no collective", "kernel_path": path,
                       "l2": "working set per step (0.40 GB at c2) exceeds the 126 MB L2; no explicit flush",
                       "algorithmic_gflop_per_step": flops / 1e9,
                       "algorithmic_gb_per_step": (fwd_bytes + bwd_bytes) / 1e9},
            "fwd_ms": fwd_t, "bwd_ms": bwd_t,
            "roofline": {"bound": "hbm", "kernel": dominant[0], "achieved": achieved, "peak": hbm_peak,
                         "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": (NCU_TRAFFIC_C2[dominant[0]] * B / 8 if args.workload == "c2" else None),
                         "peak_source": which,
                         "step_frac": ((fwd_bytes + bwd_bytes) / (ms_step * 1e-3) / 1e9) / hbm_peak,
                         "step_frac_nominal_8tbs": ((fwd_bytes + bwd_bytes) / (ms_step * 1e-3) / 1e9) / 8000.0},
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "natten_mps_b200.HostStep (batch slices over copy-in / compute / copy-out streams)",
                    "isolated_step_ms": e2e_latency_ms, "autograd_api_ms_per_step": e2e_autograd_ms},
            "gpu_launches": launches,
            "clocks": clocks.summary(),
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
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
