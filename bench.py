#!/usr/bin/env python
"""Benchmark of the LSTM forward+backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
                    [--extras NAME,NAME|none]

A step = one forward + full backward pass over one GLOBAL batch of seeded synthetic input (the reference
has no dataset; see flashlstm_poc_b200/workloads.py).  The headline workload is benchmark configuration 3
(2 layers, BF16, I=H=2048, B=256, T=1024), the configuration that covers H=2048 and the 1/2/4/8-GPU split.
With N GPUs the global batch stays 256 and rank r takes rows [r*256/N, (r+1)*256/N) ("scaling": "strong");
the weight gradients are summed with one NCCL allreduce per layer inside the backward pass.  Further
configurations are measured the same way and reported under `extra` in the same line: configuration 2
(FP16, 1 layer, I=H=1024, B=64, T=512; one GPU only) and configuration 5 (BF16, 4 layers, H=1024, B=2048,
T=256; batch-sharded like the headline).

Prints ONE JSON line (rank 0).  `value` is tokens/s (global batch * timesteps per second) with inputs
resident in HBM; `e2e` is the same metric through the engine's C ABI with pinned HOST tensors, the
host<->device copies of x, dY, y and dX inside the timed region; `roofline` describes the slower recurrent
kernel against its bound, `roofline_gemm` the dense contractions against the measured tensor peak;
`cpu_baseline` is torch.nn.LSTM (fp32) on this box's host cores on a bounded sample; `dp_check` (N > 1) compares
the reduced weight gradients with the CPU oracle and with the sum of unreduced per-rank gradients.

`--impl reference` times the reference's algorithm on the host cores (the numpy restatement of its CPU
playground under oracle/; the reference's CUDA code is a GPU program and is compared on the GPU elsewhere).
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
DEFAULT_WORKLOAD = "c3_bf16_l2_h2048"
DEFAULT_EXTRAS = "c2_fp16_h1024,c5_bf16_l4_h1024"
SHARDED = ("c3_bf16_l2_h2048", "c5_bf16_l4_h1024")  # the configurations the batch split is defined for

# DRAM bytes per launch of the recurrent kernels from ncu captures of small cases (dram__bytes_read.sum +
# dram__bytes_write.sum, summaries under profiles/).  Stored figures, not measured by this run.
STORED_TRAFFIC = {
    ("c2_fp16_h1024", "recurrent_fwd"): {"bytes_per_timestep": 1.20e6, "batch_per_gpu": 64,
                                         "source": "profiles/lstm_fwd_kernel_c2_fp16_h1024_T128.md (T=128, per step)"},
    # per-step path at 256 sequences per GPU: split-K GEMM 37.8 MB + pointwise kernel 19.9 MB per time step,
    # each launch captured cold (caches flushed); the forward kernel keeps W_hh in L2 across its steps
    ("c3_bf16_l2_h2048", "bptt"): {"bytes_per_timestep": 57.7e6, "batch_per_gpu": 256,
                                   "source": "profiles/step_kernel_c3_bf16_l2_h2048_T8.md (T=8, per time step, cold launches)"},
    ("c3_bf16_l2_h2048", "recurrent_fwd"): {"bytes_per_timestep": 12.4e6, "batch_per_gpu": 256,
                                            "source": "profiles/step_kernel_c3_bf16_l2_h2048_T8.md (wide_fwd_kernel, T=8, per time step)"},
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--extras", default=DEFAULT_EXTRAS, help="comma-separated further workloads, or 'none'")
    ap.add_argument("--backend", default="auto", choices=["auto", "simt", "tc"])
    ap.add_argument("--seq-len", type=int, default=0, help="override the workload's sequence length (profiling)")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's global batch (profiling)")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying one captured CUDA graph")
    ap.add_argument("--recompute", type=int, default=0,
                    help="activation-checkpoint interval R (0 = full gate cache, the benchmark configuration)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cudnn", action="store_true")
    ap.add_argument("--no-dp-check", action="store_true")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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


def resolve_workload(name, args):
    from flashlstm_poc_b200.workloads import WORKLOADS

    w = WORKLOADS[name]
    if args.seq_len:
        w = w.scaled(seq_len=args.seq_len, name=f"{w.name}[T={args.seq_len}]")
    if args.batch:
        w = w.scaled(batch=args.batch, name=f"{w.name}[B={args.batch}]")
    return w


def config_dict(w, world):
    """The workload description; identical in both arms so that the two lines can be matched."""
    es = 4 if w.dtype == "f32" else 2
    ws_mib = (2 if w.training else 1) * w.layers * w.seq_len * (w.batch // world) * 4 * w.hidden_size * es / 2**20
    return {"workload": w.name, "layers": w.layers, "input_size": w.input_size, "hidden_size": w.hidden_size,
            "global_batch": w.batch, "batch_per_gpu": w.batch // world, "seq_len": w.seq_len,
            "parallelism": f"dp{world}",
            "l2": "no flush: the per-GPU working set (gate cache + dG = %.0f MiB) %s" % (
                ws_mib, "exceeds the 126 MB L2" if ws_mib > 126 else "fits the 126 MB L2 (diagnostic size)")}


# ----------------------------------------------------------------------------- CPU legs
def cpu_oracle_seconds(w, sample_T: int, sample_B: int):
    """The oracle (numpy restatement of the reference's CPU playground) on the host cores: forward + backward
    over the first `sample_T` steps of the first `sample_B` sequences of the workload, full width and depth."""
    from flashlstm_poc_b200.workloads import make_inputs
    from oracle import lstm_oracle as orc

    ws = w.scaled(seq_len=sample_T, batch=sample_B)
    inp = make_inputs(ws)
    params = [orc.LayerParams(inp.w_ih[l].numpy(), inp.w_hh[l].numpy(), inp.b_ih[l].numpy(), inp.b_hh[l].numpy())
              for l in range(w.layers)]
    x = inp.x.numpy()
    h0 = None if inp.h0 is None else inp.h0.numpy()
    c0 = None if inp.c0 is None else inp.c0.numpy()
    t0 = time.perf_counter()
    fwd = orc.lstm_forward(x, params, h0, c0)
    if w.training:
        orc.lstm_backward(fwd, params, inp.dy.numpy())
    return time.perf_counter() - t0


def reference_arm(args):
    """bench.py --impl reference: the reference's algorithm (numpy port of its CPU playground) on the host cores,
    all threads.  One "step" times a bounded sample (a slice of the batch and of the sequence, full width and
    depth); the cost is linear in both, and ms_per_step is the sample time scaled to the whole step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import torch

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = resolve_workload(args.workload, args)
    # about a second of CPU work per sample: 2e11 FLOP
    sample_B = min(w.batch, 16)
    per_token = w.flops() / w.tokens
    sample_T = max(1, min(w.seq_len, int(2.0e11 / (per_token * sample_B))))
    secs = []
    for i in range(args.warmup + args.steps):
        sec = cpu_oracle_seconds(w, sample_T, sample_B)
        if i >= args.warmup:
            secs.append(sec)
    sec = statistics.median(secs)
    tps = sample_B * sample_T / sec
    ms_full = w.tokens / tps * 1e3
    sample = (f"first {sample_T} of {w.seq_len} time steps of {sample_B} of {w.batch} sequences, full width and depth, "
              f"fwd+bwd, {sec * 1e3:.0f} ms per sample; ms_per_step is the sample scaled to the whole step "
              f"(cost is linear in T and B); numpy restatement of the reference's CPU playground, BLAS on {cores} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_full, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(w, max(args.gpus, 1)),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                         "threads_env": {k: os.environ.get(k) for k in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS")}},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def cpu_torch_baseline(w):
    """torch.nn.LSTM (fp32) forward + backward on all host cores.  Workloads with more than 64 sequences are timed
    on 16 sequences at full T, width and depth and scaled linearly in the batch."""
    import torch

    from flashlstm_poc_b200.workloads import make_inputs

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample_B = w.batch if w.batch <= 64 else 16
    ws = w.scaled(batch=sample_B)
    inp = make_inputs(ws)
    m = torch.nn.LSTM(w.input_size, w.hidden_size, num_layers=w.layers)
    with torch.no_grad():
        for l in range(w.layers):
            getattr(m, f"weight_ih_l{l}").copy_(inp.w_ih[l])
            getattr(m, f"weight_hh_l{l}").copy_(inp.w_hh[l])
            getattr(m, f"bias_ih_l{l}").copy_(inp.b_ih[l])
            getattr(m, f"bias_hh_l{l}").copy_(inp.b_hh[l])
    x = inp.x.clone().requires_grad_(w.training)
    L, H = w.layers, w.hidden_size
    h0 = torch.zeros(L, sample_B, H) if inp.h0 is None else inp.h0
    c0 = torch.zeros(L, sample_B, H) if inp.c0 is None else inp.c0

    def step(T):
        if w.training:
            m.zero_grad(set_to_none=True)
            x.grad = None
            y, _ = m(x[:T], (h0, c0))
            y.backward(inp.dy[:T])
        else:
            with torch.no_grad():
                m(x[:T], (h0, c0))

    step(min(4, w.seq_len))  # warm the thread pool
    best = float("inf")
    for _ in range(2 if w.batch <= 64 else 1):
        t0 = time.perf_counter()
        step(w.seq_len)
        best = min(best, time.perf_counter() - t0)
    tps = sample_B * w.seq_len / best
    sample = (f"{sample_B} of {w.batch} sequences at full T={w.seq_len}, width and depth, fwd+bwd, {best:.2f} s"
              + ("" if sample_B == w.batch else "; extrapolated linearly in the batch"))
    return {"value": tps, "unit": UNIT, "cores": cores, "torch_threads": torch.get_num_threads(), "kind": "port",
            "impl": "torch.nn.LSTM fp32 on the host cores (the ground truth of every parity test)", "sample": sample}


# ----------------------------------------------------------------------------- GPU measurement
def recurrent_roofline(w, B, plan, phase_ms, peaks, tc):
    """Roofline entry of the slower recurrent kernel.  Per time step and layer a recurrent kernel moves
    8 H^2 bytes of W_hh (counted every step: the W_hh-streaming convention) plus 20 B H (forward: projection in,
    h in, y out, gates out), 12 B H (inference) or 22 B H (BPTT) of activations, and does 8 B H^2 FLOP;
    the bound is whichever of bytes / HBM peak and FLOP / tensor peak is longer."""
    T, H, L = w.seq_len, w.hidden_size, w.layers
    steps = T * L
    cand = [("recurrent_fwd", 8 * H * H + (20 if w.training else 12) * B * H)]
    if w.training:
        cand.append(("bptt", 8 * H * H + 22 * B * H))
    dom, dom_bytes = max(cand, key=lambda kv: phase_ms.get(kv[0], 0.0))
    dom_ms = phase_ms.get(dom, 0.0)
    us_step = dom_ms * 1e3 / steps if steps else 0.0
    flop_step = 8.0 * B * H * H
    t_hbm = dom_bytes / (peaks["hbm_gbs"] * 1e9)
    t_tensor = flop_step / (peaks["bf16_tflops"] * 1e12)
    step_path = bool(plan and plan.step_path)
    if not tc:
        kernel, per_launch_steps, launches = "simt::persistent_%s" % dom, T, L
    elif step_path and dom == "recurrent_fwd" and os.environ.get("FLSTM_WIDE_PERSIST", "1") != "0":
        kernel, per_launch_steps, launches = "tc::wide_fwd_kernel (all time steps of a layer in one launch)", T, L
    elif step_path:
        kernel = ("tc::step_kernel<LSTM_FWD> (one launch per time step)" if dom == "recurrent_fwd" else
                  "tc::step_bwd_pointwise_kernel + tc::step_kernel<F32_PARTS> (one pair per time step)")
        per_launch_steps, launches = 1, steps
    else:
        kernel, per_launch_steps, launches = ("tc::lstm_fwd_kernel" if dom == "recurrent_fwd" else "tc::lstm_bwd_kernel"), T, L
    dur_s = dom_ms * 1e-3 / max(launches, 1)
    out = {"kernel": kernel, "phase": dom, "us_per_timestep": us_step, "launches_in_phase": launches,
           "timesteps_per_launch": per_launch_steps, "algorithmic_bytes_per_timestep": dom_bytes,
           "algorithmic_flop_per_timestep": flop_step, "bound_us_per_timestep": max(t_hbm, t_tensor) * 1e6,
           "peak_source": peaks["source"], "traffic": None}
    if t_tensor > t_hbm:
        achieved = flop_step * per_launch_steps / dur_s / 1e12 if dur_s > 0 else 0.0
        out.update(bound="tensor", achieved=achieved, peak=peaks["bf16_tflops"], unit="TFLOP/s",
                   frac=achieved / peaks["bf16_tflops"])
    else:
        achieved = dom_bytes * per_launch_steps / dur_s / 1e9 if dur_s > 0 else 0.0
        out.update(bound="hbm", achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s", frac=achieved / peaks["hbm_gbs"])
    for key, name in (("traffic", dom), ("traffic_recurrent_fwd_kernel", "recurrent_fwd")):
        stored = STORED_TRAFFIC.get((w.name, name))
        if stored and stored["batch_per_gpu"] == B and (key == "traffic" or name != dom):
            steps_per_launch = per_launch_steps if name == dom else (T if tc and not (step_path and os.environ.get("FLSTM_WIDE_PERSIST", "1") == "0") else 1)
            out[key] = stored["bytes_per_timestep"] * steps_per_launch
            out[key + "_source"] = "stored figure, " + stored["source"]
    return out


def measure_workload(args, w, world, rank, dev, headline):
    """Device-resident measurement of one workload (global batch w.batch sharded over `world` ranks)."""
    import torch
    import torch.distributed as dist

    from flashlstm_poc_b200 import _lib
    from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine
    from flashlstm_poc_b200.parallel import shard_range
    from flashlstm_poc_b200.workloads import make_inputs

    td = TORCH_DTYPES[w.dtype]
    lo, hi = shard_range(w.batch, rank, world)
    inp = make_inputs(w, rows=slice(lo, hi) if world > 1 else None)
    B = hi - lo
    T, H, I, L = w.seq_len, w.hidden_size, w.input_size, w.layers
    eng = Engine(w.dtype, L, B, I, H, T, training=w.training, backend=args.backend, device=dev)
    P = [[t.to(dev) for t in (inp.w_ih[l], inp.w_hh[l], inp.b_ih[l], inp.b_hh[l])] for l in range(L)]
    for l in range(L):
        eng.set_weights(l, *P[l])
    if args.recompute:
        eng.set_recompute_interval(args.recompute)
    if world > 1:
        from flashlstm_poc_b200.parallel import attach_data_parallel

        attach_data_parallel(eng)

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

    # at N = 1 the whole step (GEMMs, recurrent kernels) is captured once and replayed
    graph, launch_mode = None, "eager launches"
    if world > 1:
        launch_mode = "eager launches (the step graph is used at N=1 only: no capture with a communicator attached)"
    elif not args.no_graph:
        try:
            graph = eng.capture_step(x, h0, c0, y, hn, cn, dy, dx, dh0, dc0)
            launch_mode = "one captured CUDA graph per step"
        except Exception as exc:  # capture is an optimisation; the eager path is the same kernels
            launch_mode = f"eager launches (graph capture failed: {type(exc).__name__})"
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

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()

    # ---- timed region: exactly K steps, CUDA events on the launching stream, max over ranks
    sampler = ClockSampler(dev.index)
    if rank == 0 and headline:
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
    clocks = sampler.stop() if (rank == 0 and headline) else None
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    tokens_per_s = w.batch * T / (ms_per_step * 1e-3)

    # ---- per-phase device time (separate eager pass with event records between the phases)
    eng.enable_timing(True)
    phase_acc = {}
    reps = 3
    for _ in range(reps):
        eager_step()
        torch.cuda.synchronize()
        for k, v in eng.phase_ms().items():
            phase_acc[k] = phase_acc.get(k, 0.0) + v / reps
    eng.enable_timing(False)
    if world > 1:  # the slowest rank's phases describe the step
        keys = sorted(phase_acc)
        t = torch.tensor([phase_acc[k] for k in keys], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        phase_acc = dict(zip(keys, [float(v) for v in t.tolist()]))

    peaks = measured_peaks()
    tc = eng.backend == "tc"
    plan = None
    if tc:
        plan = _lib.TcPlanInfo()
        if _lib.load().flstm_tc_plan(B, H, 1 if w.training else 0, 148, 232448, plan) != 0:
            plan = None
    roofline = recurrent_roofline(w, B, plan, phase_acc, peaks, tc)
    # dense contractions (projection, weight and input gradients): 2/3 of the training FLOPs (half in inference)
    gemm_flops = w.flops() / world * (2.0 / 3.0 if w.training else 0.5)
    gemm_ms = phase_acc.get("projection", 0.0) + phase_acc.get("weight_grad", 0.0) + phase_acc.get("input_grad", 0.0)
    gemm_tflops = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    roofline_gemm = None
    if tc and gemm_tflops:
        roofline_gemm = {"bound": "tensor", "kernel": "tc::gemm_kernel (projection, dW_ih, dW_hh, dX; the weight-gradient "
                         "phase includes the bias-gradient column sum)", "achieved": gemm_tflops, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": gemm_tflops / peaks["bf16_tflops"], "frac_of_nominal_2250": gemm_tflops / 2250.0,
                         "peak_source": peaks["source"] + " (burst)", "per_gemm_tflops": {
                             "projection": w.flops() / world / 6 / (phase_acc["projection"] * 1e-3) / 1e12 if phase_acc.get("projection") else None,
                             "input_grad": w.flops() / world / 6 / (phase_acc["input_grad"] * 1e-3) / 1e12 if phase_acc.get("input_grad") else None,
                             "weight_grad": w.flops() / world / 3 / (phase_acc["weight_grad"] * 1e-3) / 1e12 if phase_acc.get("weight_grad") else None}}
    res = {
        "tokens_per_s": tokens_per_s, "ms_per_step": ms_per_step, "launches": launches, "launch_mode": launch_mode,
        "phase_ms": {k: round(v, 4) for k, v in phase_acc.items()}, "roofline": roofline, "roofline_gemm": roofline_gemm,
        "mfu_vs_measured_bf16_sustained": w.flops() / world / (ms_per_step * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12),
        "mfu_vs_nominal_2250": w.flops() / world / (ms_per_step * 1e-3) / 2250e12,
        "backend": eng.backend, "recurrent_path": ("per-step GEMM launches" if (plan and plan.step_path) else "persistent kernels") if tc else "simt",
        "workspace_gib": eng.workspace_bytes / 2**30, "clocks": clocks, "warmup": warmup,
    }

    # ---- end to end with host buffers
    if not args.no_e2e and w.training and not args.recompute:
        res["e2e"] = run_e2e_engine(args, eng, w, inp, B, dev, td, world, (x, dy, y, dx, h0, c0, hn, cn, dh0, dc0))
        if w.layers == 1 and w.dtype == "f16" and world == 1:
            res["e2e_reference_surface"] = run_e2e_v2(args, w, inp, dev)

    # ---- on-GPU comparison: cuDNN through torch.nn.LSTM in the workload's dtype (what the reference's own
    # benchmark compares itself with, python/benchmark_lstm.py:304-328); baseline code only
    if rank == 0 and world == 1 and not args.no_cudnn:
        del x, dy, y, dx
        try:
            res["cudnn_torch_nn_lstm"] = cudnn_tokens_per_sec(w, inp, dev, td)
        except Exception as exc:
            res["cudnn_torch_nn_lstm"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
        torch.cuda.empty_cache()

    # ---- N > 1: the reduced gradients against the oracle and against the sum of the unreduced ones
    if world > 1 and headline and w.training and not args.no_dp_check:
        res["dp_check"] = dp_check(args, eng, w, inp, P, B, dev, td, world, rank)
    eng.close()
    torch.cuda.empty_cache()
    return res


def cudnn_tokens_per_sec(w, inp, dev, td, iters=5):
    """torch.nn.LSTM on the same device (cuDNN), same weights / inputs / dtype, forward + backward."""
    import torch

    m = torch.nn.LSTM(w.input_size, w.hidden_size, num_layers=w.layers).to(dev, td)
    with torch.no_grad():
        for l in range(w.layers):
            getattr(m, f"weight_ih_l{l}").copy_(inp.w_ih[l])
            getattr(m, f"weight_hh_l{l}").copy_(inp.w_hh[l])
            getattr(m, f"bias_ih_l{l}").copy_(inp.b_ih[l])
            getattr(m, f"bias_hh_l{l}").copy_(inp.b_hh[l])
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


def run_e2e_engine(args, eng, w, inp, B, dev, td, world, bufs, chunks=8):
    """The step through flstm_engine_forward_range / flstm_engine_backward_range with pinned HOST x, dY, y, dX:
    every step copies its inputs host->device and its results device->host, chunk by chunk on side streams so
    that the copies overlap the ranges already enqueued (what the reference's v2 does with its 32-step chunks,
    flashlstm_v2/src/lstm_forward.cu:673-940)."""
    import torch
    import torch.distributed as dist

    x_d, dy_d, y_d, dx_d, h0, c0, hn, cn, dh0, dc0 = bufs
    T = w.seq_len
    x_h = inp.x.to(td).pin_memory()
    dy_h = inp.dy.to(td).pin_memory()
    y_h = torch.empty(T, B, w.hidden_size, dtype=td).pin_memory()
    dx_h = torch.empty(T, B, w.input_size, dtype=td).pin_memory()
    s_c = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    n = min(chunks, T)
    bounds = [(k * T // n, (k + 1) * T // n) for k in range(n)]
    ev_x = [torch.cuda.Event() for _ in bounds]
    ev_dy = [torch.cuda.Event() for _ in bounds]
    ev_c = [torch.cuda.Event() for _ in range(2 * n)]
    ev_step, ev_y_out, ev_dx_out = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
    ev_y_out.record(s_out)
    ev_dx_out.record(s_out)

    def step():
        ev_step.record(s_c)          # the previous step is done with the device buffers
        s_in.wait_event(ev_step)
        s_c.wait_event(ev_y_out)     # ... and its y has left the device buffer this step overwrites
        with torch.cuda.stream(s_in):
            for k, (a, b) in enumerate(bounds):
                x_d[a:b].copy_(x_h[a:b], non_blocking=True)
                ev_x[k].record(s_in)
            for k, (a, b) in reversed(list(enumerate(bounds))):
                dy_d[a:b].copy_(dy_h[a:b], non_blocking=True)
                ev_dy[k].record(s_in)
        for k, (a, b) in enumerate(bounds):
            s_c.wait_event(ev_x[k])
            eng.forward_range_into(T, a, b, x_d, h0, c0, y_d, hn, cn)
            ev_c[k].record(s_c)
            s_out.wait_event(ev_c[k])
            with torch.cuda.stream(s_out):
                y_h[a:b].copy_(y_d[a:b], non_blocking=True)
        ev_y_out.record(s_out)
        s_c.wait_event(ev_dx_out)    # the previous step's dX has left its device buffer
        for k, (a, b) in reversed(list(enumerate(bounds))):
            s_c.wait_event(ev_dy[k])
            eng.backward_range_into(T, a, b, dy_d, None, None, dx_d, dh0, dc0)
            ev_c[n + k].record(s_c)
            s_out.wait_event(ev_c[n + k])
            with torch.cuda.stream(s_out):
                dx_h[a:b].copy_(dx_d[a:b], non_blocking=True)
        ev_dx_out.record(s_out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(2):
        step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()  # all three streams
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    barrier()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    es = x_h.element_size()
    return {"value": w.batch * T / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms,
            "h2d_bytes_per_step": (x_h.numel() + dy_h.numel()) * es, "d2h_bytes_per_step": (y_h.numel() + dx_h.numel()) * es,
            "bytes_are": "per rank" if world > 1 else "whole job",
            "api": f"flstm_engine_forward_range / flstm_engine_backward_range (C ABI) over {n} time chunks, pinned host "
                   "x / dY / y / dX, copies on side streams inside the timed region; timed with the host clock around "
                   "synchronised steps"}


def run_e2e_v2(args, w, inp, dev):
    """The reference's own surface: flstm_StreamingLstmForward + flstm_StreamingLstmBackward with pinned host
    x / y / dY / dx and checkpoint tensors (single layer, FP16 only: what that surface can express)."""
    import torch

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
    P = [t.to(dev).contiguous() for t in (inp.w_ih[0], inp.w_hh[0], inp.b_ih[0], inp.b_hh[0])]
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

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / args.steps  # the calls are synchronous: the host clock is the honest one
    h2d = x.numel() * 2 + dy.numel() * 2
    d2h = y.numel() * 2 + dx.numel() * 2 + ch.numel() * 2 + cc.numel() * 4
    return {"value": B * T / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h,
            "api": "flstm_StreamingLstmForward + flstm_StreamingLstmBackward (the reference's C ABI, pinned host tensors, R=1)"}


def dp_check(args, eng, w, inp, P, B, dev, td, world, rank):
    """Gradient parity of the batch split.  One extra step in which dY is zero except for a few sequences per rank
    (a sequence whose dY is zero contributes nothing to dW and db), so that the reduced gradients can be
    compared with the CPU oracle run on just those sequences; and the same step on a second engine WITHOUT a
    communicator, whose per-rank gradients are summed over the ranks with torch.distributed and compared with
    what the engine's own in-backward allreduce produced."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from flashlstm_poc_b200.engine import Engine
    from oracle import lstm_oracle as orc

    H, I, L = w.hidden_size, w.input_size, w.layers
    # the first 128 time steps: enough BPTT depth for the check, and the CPU oracle (memory-bound on the weights
    # at a handful of sequences) stays within tens of seconds
    T = min(w.seq_len, 128)
    rows = list(range(max(1, 4 // world)))  # local rows whose dY is kept
    x = inp.x[:T].to(dev, td)
    dy = torch.zeros(T, B, H, dtype=td, device=dev)
    dy[:, rows] = inp.dy[:T, rows].to(dev, td)
    eng.forward_into(T, x, None, None, None, None, None)
    eng.backward_into(T, dy, None, None, None, None, None)
    torch.cuda.synchronize()
    reduced = [[g.clone() for g in eng.grads(l)] for l in range(L)]
    solo = Engine(w.dtype, L, B, I, H, T, training=True, backend=args.backend, device=dev)
    for l in range(L):
        solo.set_weights(l, *P[l])
    solo.forward_into(T, x, None, None, None, None, None)
    solo.backward_into(T, dy, None, None, None, None, None)
    torch.cuda.synchronize()
    worst_sum = 0.0
    for l in range(L):
        for got, loc in zip(reduced[l], solo.grads(l)):
            tot = loc.clone()
            dist.all_reduce(tot)
            err = float((got - tot).norm() / tot.norm().clamp_min(1e-30))
            worst_sum = max(worst_sum, err)
    solo.close()
    # every rank sends its kept sequences to rank 0, which runs the oracle on all of them
    xs = [torch.empty(T, len(rows), I, dtype=td, device=dev) for _ in range(world)]
    dys = [torch.empty(T, len(rows), H, dtype=td, device=dev) for _ in range(world)]
    dist.all_gather(xs, x[:, rows].contiguous())
    dist.all_gather(dys, dy[:, rows].contiguous())
    worst_oracle, oracle_s = None, None
    if rank == 0:
        t0 = time.perf_counter()
        params = [orc.LayerParams(inp.w_ih[l].numpy(), inp.w_hh[l].numpy(), inp.b_ih[l].numpy(), inp.b_hh[l].numpy())
                  for l in range(L)]
        # the launcher pins every rank to one BLAS thread; the other ranks idle while rank 0 runs the oracle
        try:
            from threadpoolctl import threadpool_limits
            blas_threads = threadpool_limits(limits=os.cpu_count() or 1)
        except Exception:
            blas_threads = None
        fwd = orc.lstm_forward(torch.cat(xs, 1).float().cpu().numpy(), params, None, None)
        bwd = orc.lstm_backward(fwd, params, torch.cat(dys, 1).float().cpu().numpy())
        if blas_threads is not None:
            blas_threads.restore_original_limits()
        oracle_s = time.perf_counter() - t0
        worst_oracle = 0.0
        for l in range(L):
            for got, want in zip(reduced[l], (bwd.dw_ih[l], bwd.dw_hh[l], bwd.db_ih[l])):
                worst_oracle = max(worst_oracle, float(orc.rel_l2_err(got.float().cpu().numpy(), want)))
    flag = torch.tensor([0.0 if worst_oracle is None else worst_oracle], device=dev)
    dist.broadcast(flag, 0)
    worst_oracle = float(flag.item())
    ok = worst_oracle <= 1e-2 and worst_sum <= 1e-4
    return {"ok": bool(ok), "tensors": "dW_ih, dW_hh, db of every layer",
            "rel_l2_vs_cpu_oracle": worst_oracle, "tolerance_vs_oracle": 1e-2,
            "rel_l2_vs_sum_of_unreduced_rank_gradients": worst_sum, "tolerance_vs_sum": 1e-4,
            "sequences_with_nonzero_dY": len(rows) * world, "time_steps": T, "oracle_seconds": oracle_s,
            "note": "dY is zero for all other sequences of this check step, so they add nothing to dW / db"}


# ----------------------------------------------------------------------------- our arm
def main():
    args = parse_args()
    if args.impl == "reference":
        # a launcher may export OMP_NUM_THREADS=1; the CPU arm uses every host core
        cores = str(os.cpu_count() or 1)
        for k in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
            os.environ[k] = cores
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = resolve_workload(args.workload, args)
    if world > 1 and w.batch % world:
        raise SystemExit(f"global batch {w.batch} does not divide over {world} ranks")
    head = measure_workload(args, w, world, rank, dev, headline=True)

    extra = {}
    names = [] if args.extras in ("", "none") else [n for n in args.extras.split(",") if n and n != args.workload]
    for name in names:
        we = resolve_workload(name, args) if not (args.seq_len or args.batch) else None
        if we is None:
            continue  # overrides are for profiling the headline workload alone
        if world > 1 and (name not in SHARDED or we.batch % world):
            extra[name] = {"skipped": "measured on one GPU only (the batch split is defined for configurations 3 and 5)"}
            continue
        try:
            r = measure_workload(args, we, world, rank, dev, headline=False)
            r["config"] = config_dict(we, world)
            r.pop("clocks", None)
            extra[name] = r
        except Exception as exc:  # an extra never takes the headline line down
            extra[name] = {"failed": f"{type(exc).__name__}: {exc}"[:300]}
            torch.cuda.synchronize()

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = cpu_torch_baseline(w)

    if rank == 0:
        e2e = head.pop("e2e", None)
        line = {
            "metric": METRIC, "value": head.pop("tokens_per_s"), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": head.pop("warmup"), "ms_per_step": head.pop("ms_per_step"), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": config_dict(w, world), "clocks": head.pop("clocks"), "e2e": e2e,
            "gpu_launches": head.pop("launches"), "roofline": head.pop("roofline"),
            "roofline_gemm": head.pop("roofline_gemm"), "cpu_baseline": cpu_baseline, **head, "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
