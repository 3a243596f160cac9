"""Per-time-step clock trace of the persistent recurrent kernels (tensor-core backend).

    python -m flashlstm_poc_b200.step_trace [workload-name] [--steps N] [--batch B] [--seq-len T]

CTA 0 of the forward and of the BPTT kernel stamps clock64() at fixed points of each of the first N time steps
(flstm_engine_enable_trace / flstm_engine_read_trace in include/flashlstm_b200/engine.h).  `trace_report`
prints, per point, the median distance in SM cycles from the same CTA's release of the previous step: where a
step's time goes.  The role of the reference's NVTX ranges and MFU printer (flashlstm_v2/src/gputx.h:27-60,
flashlstm_v2/include/mfu_profiler.hpp:24-98) for kernels that run a whole sequence in one launch."""
from __future__ import annotations

import argparse
import ctypes
from typing import Dict

import numpy as np
import torch

from ._lib import check
from .engine import TORCH_DTYPES, Engine
from .workloads import WORKLOADS, make_inputs

POINTS = {0: "step barrier satisfied", 1: "TMA copies issued", 2: "first chunk landed", 3: "last chunk landed",
          4: "last UMMA committed", 5: "epilogue sees the accumulator", 9: "partial sums sent (BPTT)",
          10: "reduce-scatter complete (BPTT)", 6: "accumulator exchanged", 7: "state stores issued", 8: "released"}
ORDER = {"forward": (0, 1, 2, 3, 4, 5, 6, 7, 8), "bptt": (0, 1, 2, 3, 4, 5, 9, 10, 6, 7, 8)}


def collect(engine: Engine, run_step, steps: int = 64) -> np.ndarray:
    """Stamps of one traced step: array [2 (forward, BPTT)][steps][16] of clock64() values (0 = point not hit).
    `run_step()` must enqueue one forward + backward on `engine`."""
    check(engine.lib.flstm_engine_enable_trace(engine._h, steps))
    run_step()
    torch.cuda.synchronize(engine.device)
    buf = (ctypes.c_longlong * (2 * steps * 16))()
    check(engine.lib.flstm_engine_read_trace(engine._h, buf, 2 * steps * 16))
    check(engine.lib.flstm_engine_enable_trace(engine._h, 0))
    return np.array(buf[:], dtype=np.int64).reshape(2, steps, 16)


def summarize(stamps: np.ndarray, skip: int = 10) -> Dict[str, Dict[str, float]]:
    """Median cycles from the previous step's release to each point, per kernel; 'period' = release to release."""
    out = {}
    for d, name in enumerate(("forward", "bptt")):
        t = stamps[d]
        if t[skip:, 8].min() == 0:
            continue
        rel = t[skip:-1, 8]  # release of the previous step
        rows = {"period": float(np.median(np.diff(t[skip:, 8])))}
        for k in ORDER[name]:
            v = t[skip + 1:, k]
            if v.min() == 0:
                continue
            rows[POINTS[k]] = float(np.median(v - rel))
        out[name] = rows
    return out


def trace_report(workload: str = "c2_fp16_h1024", steps: int = 64, **scale) -> Dict[str, Dict[str, float]]:
    """`scale` (batch=, seq_len=, ...) shrinks the named workload, e.g. to one GPU's shard of its batch."""
    w = WORKLOADS[workload]
    if scale:
        w = w.scaled(**scale)
    inp = make_inputs(w)
    dev = torch.device("cuda", torch.cuda.current_device())
    td = TORCH_DTYPES[w.dtype]
    eng = Engine(w.dtype, w.layers, w.batch, w.input_size, w.hidden_size, w.seq_len, device=dev)
    for l in range(w.layers):
        eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
    x, dy = inp.x.to(dev, td), inp.dy.to(dev, td)
    h0 = None if inp.h0 is None else inp.h0.to(dev, td)
    c0 = None if inp.c0 is None else inp.c0.to(dev, td)

    def run_step():
        eng.forward(x, h0, c0)
        eng.backward(dy)

    for _ in range(3):
        run_step()
    summary = summarize(collect(eng, run_step, steps))
    eng.close()
    for name, rows in summary.items():
        print(f"{name}: step period {rows['period']:.0f} cycles")
        for point, cycles in rows.items():
            if point != "period":
                print(f"  {point:>34}: {cycles:8.0f}")
    return summary


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", nargs="?", default="c2_fp16_h1024")
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--seq-len", type=int, default=0)
    a = ap.parse_args()
    scale = {k: v for k, v in (("batch", a.batch), ("seq_len", a.seq_len)) if v > 0}
    trace_report(a.workload, a.steps, **scale)
