#!/usr/bin/env python
"""Benchmark of the LSTM forward+backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step = one forward + full backward pass over one batch of seeded synthetic input (the
reference has no dataset; see flashlstm_poc_b200/workloads.py).  At N=1 the workload is benchmark
configuration 2 (1 layer, FP16, I=H=1024, B=64, T=512).  At N>1 every rank runs that per-GPU
batch (weak scaling: global batch 64*N) and the weight gradients are summed with one NCCL
allreduce per layer inside the backward pass.

Prints ONE JSON line (rank 0).  `value` is tokens/s (batch*timesteps per second) over all
ranks with inputs resident in HBM; `e2e` is the same metric through the reference-facing C ABI
(flstm_StreamingLstmForward/Backward) with pinned HOST tensors, copies inside the timed region;
`roofline` describes the dominant kernel against the measured HBM peak; `cpu_baseline` is the CPU
oracle timed on this box's host cores on a bounded sample.

`--impl reference` times the reference's algorithm on the host cores (the oracle port: the
reference's CUDA code cannot be built here and its CPU playground needs the reference checkout).
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "lstm_fwd_bwd_tokens_per_sec"
UNIT = "tokens/s"
DEFAULT_WORKLOAD = "c2_fp16_h1024"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--backend", default="auto", choices=["auto", "simt", "tc"])
    ap.add_argument("--seq-len", type=int, default=0, help="override the workload's sequence length (profiling)")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's per-GPU batch (profiling)")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying one captured CUDA graph")
    ap.add_argument("--recompute", type=int, default=0,
                    help="activation-checkpoint interval R (0 = full gate cache, the benchmark configuration)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cudnn", action="store_true")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def resolve_workload(args):
    from flashlstm_poc_b200.workloads import WORKLOADS

    w = WORKLOADS[args.workload]
    if args.seq_len:
        w = w.scaled(seq_len=args.seq_len, name=f"{w.name}[T={args.seq_len}]")
    if args.batch:
        w = w.scaled(batch=args.batch, name=f"{w.name}[B={args.batch}]")
    return w


# ----------------------------------------------------------------------------- CPU legs
def cpu_oracle_tokens_per_sec(w, sample_T: int, repeats: int = 1):
    """The oracle (numpy restatement of the reference's algorithm) on the host cores, on the first
    `sample_T` time steps of the workload at full batch and width."""
    import numpy as np

    from flashlstm_poc_b200.workloads import make_inputs
    from oracle import lstm_oracle as orc

    ws = w.scaled(seq_len=sample_T)
    inp = make_inputs(ws)
    params = [orc.LayerParams(inp.w_ih[l].numpy(), inp.w_hh[l].numpy(), inp.b_ih[l].numpy(), inp.b_hh[l].numpy())
              for l in range(w.layers)]
    x = inp.x.numpy()
    h0 = None if inp.h0 is None else inp.h0.numpy()
    c0 = None if inp.c0 is None else inp.c0.numpy()
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fwd = orc.lstm_forward(x, params, h0, c0)
        if w.training:
            orc.lstm_backward(fwd, params, inp.dy.numpy())
        best = min(best, time.perf_counter() - t0)
    return ws.batch * ws.seq_len / best, best


def reference_arm(args):
    """bench.py --impl reference: the reference's algorithm on the host cores, all threads."""
    import torch

    from flashlstm_poc_b200.workloads import WORKLOADS

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    w = resolve_workload(args)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample_T = min(w.seq_len, 128)
    per_step = []
    for i in range(args.warmup + args.steps):
        tps, sec = cpu_oracle_tokens_per_sec(w, sample_T)
        if i >= args.warmup:
            per_step.append((tps, sec))
    tps = statistics.median(t for t, _ in per_step)
    ms = statistics.median(s for _, s in per_step) * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "layers": w.layers, "input_size": w.input_size, "hidden_size": w.hidden_size,
                   "batch": w.batch, "seq_len": w.seq_len},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"first {sample_T} of {w.seq_len} time steps at full batch/width, fwd+bwd, "
                                   f"numpy (multi-threaded BLAS) restatement of the reference's CPU playground"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------- our arm
def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from flashlstm_poc_b200 import _lib
    from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine
    from flashlstm_poc_b200.workloads import WORKLOADS, make_inputs

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = resolve_workload(args)
    td = TORCH_DTYPES[w.dtype]
    inp = make_inputs(w.scaled(seed=w.seed + rank))  # every rank owns different sequences (weak scaling)
    base = make_inputs(w) if rank else inp            # weights are replicated: rank 0's draw
    eng = Engine(w.dtype, w.layers, w.batch, w.input_size, w.hidden_size, w.seq_len, training=w.training,
                 backend=args.backend, device=dev)
    for l in range(w.layers):
        eng.set_weights(l, base.w_ih[l].to(dev), base.w_hh[l].to(dev), base.b_ih[l].to(dev), base.b_hh[l].to(dev))
    if args.recompute:
        eng.set_recompute_interval(args.recompute)
    if world > 1:
        from flashlstm_poc_b200.parallel import attach_data_parallel

        attach_data_parallel(eng)

    T, B, H, I, L = w.seq_len, w.batch, w.hidden_size, w.input_size, w.layers
    x = inp.x.to(dev, td)
    h0 = None if inp.h0 is None else inp.h0.to(dev, td)
    c0 = None if inp.c0 is None else inp.c0.to(dev, td)
    dy = inp.dy.to(dev, td) if w.training else None
    y = torch.empty(T, B, H, dtype=td, device=dev)
    hn = torch.empty(L, B, H, dtype=td, device=dev)
    cn = torch.empty(L, B, H, dtype=td, device=dev)
    dx = torch.empty(T, B, I, dtype=td, device=dev) if w.training else None
    dh0 = torch.empty(L, B, H, dtype=torch.float32, device=dev) if w.training else None
    dc0 = torch.empty(L, B, H, dtype=torch.float32, device=dev) if w.training else None

    def eager_step():
        eng.forward_into(T, x, h0, c0, y, hn, cn)
        if w.training:
            eng.backward_into(T, dy, None, None, dx, dh0, dc0)

    # the whole step (GEMMs, persistent kernels, allreduce) is captured once and replayed
    graph, graph_note = None, "eager launches"
    if world > 1:
        # capturing the in-backward NCCL allreduce together with the cooperative kernels hung once at
        # N=2; multi-GPU runs therefore launch eagerly (same kernels, same allreduce)
        graph_note = "eager launches (graph capture is used at N=1 only)"
    elif not args.no_graph:
        try:
            graph = eng.capture_step(x, h0, c0, y, hn, cn, dy, dx, dh0, dc0)
            graph_note = "one captured CUDA graph per step"
        except Exception as exc:  # capture is an optimisation; the eager path is the same kernels
            graph_note = f"eager launches (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()
    step = graph.replay if graph is not None else eager_step
    l0 = eng.launch_count
    eager_step()
    launches_per_step = eng.launch_count - l0
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- timed region: exactly K steps, CUDA events on the launching stream
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = eng.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    total_ms = ev0.elapsed_time(ev1)
    launches = (eng.launch_count - launches0) if graph is None else launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    tokens_per_s = world * B * T / (ms_per_step * 1e-3)

    # ---- per-phase device time (separate pass with event records between phases)
    eng.enable_timing(True)
    phase_acc = {}
    reps = 3
    for _ in range(reps):
        eager_step()
        torch.cuda.synchronize()
        for k, v in eng.phase_ms().items():
            phase_acc[k] = phase_acc.get(k, 0.0) + v / reps
    eng.enable_timing(False)

    peaks = measured_peaks()
    steps_seq = T * L
    fwd_bytes_step = 8 * H * H + (20 if w.training else 12) * B * H
    bwd_bytes_step = 8 * H * H + 22 * B * H
    tc = eng.backend == "tc"
    cand = [("recurrent_fwd", fwd_bytes_step)]
    if w.training:
        cand.append(("bptt", bwd_bytes_step))
    dom, dom_bytes = max(cand, key=lambda kv: phase_acc.get(kv[0], 0.0))
    dom_ms = phase_acc.get(dom, 0.0)
    # one launch of the persistent kernel covers T steps of one layer; the SIMT path launches per step
    launches_in_phase = L if tc else steps_seq
    bytes_per_launch = dom_bytes * (T if tc else 1)
    dur_s = dom_ms * 1e-3 / max(launches_in_phase, 1)
    achieved = bytes_per_launch / dur_s / 1e9 if dur_s > 0 else 0.0
    roofline = {
        "bound": "hbm", "kernel": ("tc_" if tc else "simt_") + dom, "achieved": achieved, "peak": peaks["hbm_gbs"],
        "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"], "traffic": None,
        "us_per_timestep": dom_ms * 1e3 / steps_seq,
        "algorithmic_bytes_per_timestep": dom_bytes,
    }
    if tc and w.name.startswith("c2_fp16_h1024"):
        # DRAM bytes of the persistent forward kernel from its ncu capture (1.20 MB per time step at T=128, scaled
        # by T: the traffic is per step); the BPTT kernel cannot be replayed by ncu (cooperative + cluster launch)
        fwd_traffic = 1.20e6 * T
        if dom == "recurrent_fwd":
            roofline["traffic"] = fwd_traffic
        else:
            roofline["traffic_recurrent_fwd_kernel"] = fwd_traffic
            roofline["traffic_note"] = "no ncu capture of the BPTT kernel exists (ncu cannot replay its launch)"
    gemm_flops = w.flops() * (2.0 / 3.0 if w.training else 0.5)
    gemm_ms = phase_acc.get("projection", 0.0) + phase_acc.get("weight_grad", 0.0) + phase_acc.get("input_grad", 0.0)
    extra = {
        "phase_ms": {k: round(v, 4) for k, v in phase_acc.items()},
        "mfu_vs_measured_bf16_peak": w.flops() / (ms_per_step * 1e-3) / (peaks["bf16_tflops"] * 1e12),
        "dense_gemm_tflops": gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None,
        "backend": eng.backend,
        "recompute_interval": args.recompute,
        "workspace_gib": eng.workspace_bytes / 2**30,
    }

    # ---- end to end through the reference-facing C ABI with host buffers
    e2e = None
    if not args.no_e2e and w.layers == 1 and w.dtype == "f16" and w.training:
        e2e = run_e2e(args, w, inp, base, dev, world, rank)

    # on-GPU comparison: cuDNN through torch.nn.LSTM in the config's dtype (what the reference's own
    # benchmark compares itself with, python/benchmark_lstm.py:304-328); test/baseline code only
    cudnn = None
    if rank == 0 and world == 1 and not args.no_cudnn:
        try:
            cudnn = cudnn_tokens_per_sec(w, base, inp, dev, td)
        except Exception as exc:
            cudnn = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    extra["cudnn_torch_nn_lstm"] = cudnn

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        sample_T = T  # the whole sequence: a few seconds per pass on the host cores
        cpu_oracle_tokens_per_sec(w, 2)  # warm the BLAS threads
        tps, sec = cpu_oracle_tokens_per_sec(w, sample_T, repeats=2)
        cpu_baseline = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"all {sample_T} time steps at full batch/width, fwd+bwd, best of 2 passes "
                                  f"({sec:.2f} s each); numpy restatement of the reference's CPU playground"}

    es = 4 if w.dtype == "f32" else 2
    ws_mib = (2 if w.training else 1) * L * T * B * 4 * H * es / 2**20
    l2_note = (f"working set (gate cache{' + dG' if w.training else ''} = {ws_mib:.0f} MiB) "
               + ("exceeds the 126 MB L2" if ws_mib > 126 else "fits the 126 MB L2 (diagnostic size, not a bench configuration)"))
    if rank == 0:
        line = {
            "metric": METRIC, "value": tokens_per_s, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": {"workload": w.name, "layers": L, "input_size": I, "hidden_size": H, "batch_per_gpu": B,
                       "global_batch": B * world, "seq_len": T, "parallelism": f"dp{world}",
                       "launch": graph_note,
                       "l2": l2_note},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline,
            "cpu_baseline": cpu_baseline, **extra,
        }
        print(json.dumps(line), flush=True)
    eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def cudnn_tokens_per_sec(w, base, inp, dev, td, iters=5):
    """torch.nn.LSTM on the same device (cuDNN), same weights / inputs / dtype, forward + backward."""
    import torch

    m = torch.nn.LSTM(w.input_size, w.hidden_size, num_layers=w.layers).to(dev, td)
    with torch.no_grad():
        for l in range(w.layers):
            getattr(m, f"weight_ih_l{l}").copy_(base.w_ih[l])
            getattr(m, f"weight_hh_l{l}").copy_(base.w_hh[l])
            getattr(m, f"bias_ih_l{l}").copy_(base.b_ih[l])
            getattr(m, f"bias_hh_l{l}").copy_(base.b_hh[l])
    x = inp.x.to(dev, td).requires_grad_(w.training)
    L, B, H = w.layers, w.batch, w.hidden_size
    h0 = (torch.zeros(L, B, H) if inp.h0 is None else inp.h0).to(dev, td)
    c0 = (torch.zeros(L, B, H) if inp.c0 is None else inp.c0).to(dev, td)
    dy = inp.dy.to(dev, td) if w.training else None

    def step():
        if w.training:
            m.zero_grad(set_to_none=True)
            x.grad = None
            y, _ = m(x, (h0, c0))
            y.backward(dy)
        else:
            with torch.no_grad():
                m(x, (h0, c0))

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    return {"value": w.batch * w.seq_len / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms,
            "note": "torch.nn.LSTM (cuDNN) on the same GPU, same dtype, fwd+bwd" if w.training else
                    "torch.nn.LSTM (cuDNN) on the same GPU, same dtype, forward only"}


def run_e2e(args, w, inp, base, dev, world, rank):
    """flstm_StreamingLstmForward + flstm_StreamingLstmBackward with pinned host x / y / dY / dx and
    checkpoint tensors: every step copies its inputs host->device and its results device->host."""
    import torch
    import torch.distributed as dist

    from flashlstm_poc_b200 import _lib

    lib = _lib.load()
    T, B, H, I = w.seq_len, w.batch, w.hidden_size, w.input_size
    pin = lambda t: t.contiguous().pin_memory()
    x = pin(inp.x.half())
    dy = pin(inp.dy.half())
    y = torch.empty(T, B, H, dtype=torch.float16).pin_memory()
    dx = torch.empty(T, B, I, dtype=torch.float16).pin_memory()
    ch = torch.empty(T, B, H, dtype=torch.float16).pin_memory()
    cc = torch.empty(T, B, H, dtype=torch.float32).pin_memory()
    zeros = torch.zeros(B, H, dtype=torch.float16, device=dev)
    h0 = zeros if inp.h0 is None else inp.h0[0].to(dev, torch.float16)
    c0 = zeros if inp.c0 is None else inp.c0[0].to(dev, torch.float16)
    P = [t.to(dev).contiguous() for t in (base.w_ih[0], base.w_hh[0], base.b_ih[0], base.b_hh[0])]
    G = [torch.empty_like(p) for p in P]
    hy, cy = torch.empty_like(h0), torch.empty_like(h0)
    dh0, dc0 = torch.empty(B, H, device=dev), torch.empty(B, H, device=dev)
    s1, s2, s3 = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    opt = _lib.StreamingLstmOptions(1, 0)
    cache = _lib.GateCacheHost(ch.data_ptr(), cc.data_ptr())
    R = 1

    def step():
        lib.flstm_StreamingLstmForward(T, B, I, H, R, x.data_ptr(), h0.data_ptr(), c0.data_ptr(), P[0].data_ptr(),
                                       P[1].data_ptr(), P[2].data_ptr(), P[3].data_ptr(), y.data_ptr(), cache,
                                       ctypes.byref(opt), hy.data_ptr(), cy.data_ptr(), s1.cuda_stream,
                                       s2.cuda_stream, s3.cuda_stream)
        lib.flstm_StreamingLstmBackward(T, B, I, H, R, x.data_ptr(), y.data_ptr(), cache, dy.data_ptr(), None, None,
                                        h0.data_ptr(), c0.data_ptr(), P[0].data_ptr(), P[1].data_ptr(),
                                        P[2].data_ptr(), P[3].data_ptr(), dx.data_ptr(), G[0].data_ptr(),
                                        G[1].data_ptr(), G[2].data_ptr(), G[3].data_ptr(), dh0.data_ptr(),
                                        dc0.data_ptr(), s1.cuda_stream, s2.cuda_stream, s3.cuda_stream,
                                        ctypes.byref(opt))
        if lib.flstm_last_status() != 0:
            raise RuntimeError(lib.flstm_last_error().decode())
        if world > 1:
            for g in G[:3]:
                dist.all_reduce(g)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(3):
        step()
    barrier()
    t0 = time.perf_counter()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    # the calls are synchronous on their own streams, so the host clock around them is the honest
    # end-to-end time; the event pair on the current stream only brackets it
    ms = max(wall_ms, ev0.elapsed_time(ev1)) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    h2d = x.numel() * 2 + dy.numel() * 2
    d2h = y.numel() * 2 + dx.numel() * 2 + ch.numel() * 2 + cc.numel() * 4
    return {"value": world * B * T / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h,
            "api": "flstm_StreamingLstmForward + flstm_StreamingLstmBackward (C ABI, pinned host tensors)"}


if __name__ == "__main__":
    sys.exit(main())
