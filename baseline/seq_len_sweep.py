"""Sequence-length sweep of the reference's own benchmark, on this GPU: B=32, I=H=1024, forward only, fp32 in/out,
T from 64 to 8192 (python/benchmark_lstm.py:513-523,536-685 sweeps 64..8192 in steps of 128; a subset of that grid
is timed here), comparing
    * the rebuilt reference v1 library (baseline/_ref/libflashlstm_v1.so, see build_reference.py), FP16_ACC16 as
      the reference's benchmark requests, chunk size 64 (its stated optimum, src/run_lstm.cu:206) and 0,
    * this repository's library through the SAME C ABI and harness,
    * torch.nn.LSTM on CUDA (cuDNN, fp16: the reference's "PyTorch nn.LSTM (cuDNN)" curve, :304-328),
and, at one shape, the v2 forward+backward entry points of both libraries (configuration 2 of the benchmark:
FP16, B=64, I=H=1024, T=512, R=1).  No FlashAttention curve and no plot.  Every result is checked against fp32 CPU
torch.nn.LSTM on a short prefix before it is timed.

    python -m baseline.seq_len_sweep [--out seq_len_sweep.md] [--lengths 64,192,...]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from baseline import reference_gpu as rg  # noqa: E402


def check_v1(lib, name, lstm, B, I, H):
    """Parity of a v1 library on a short sequence against fp32 CPU torch.nn.LSTM (the reference's own check,
    python/test_lstm.py:99-105,370-381: atol 1e-3, rtol 5e-2)."""
    T = 16
    torch.manual_seed(5)
    x, h0, c0 = torch.randn(T, B, I), torch.randn(B, H), torch.randn(B, H)
    with torch.no_grad():
        y_ref, (hn_ref, cn_ref) = lstm(x, (h0.unsqueeze(0), c0.unsqueeze(0)))
    r = rg.V1Runner(lib, T, B, I, H, [lstm.weight_ih_l0, lstm.weight_hh_l0, lstm.bias_ih_l0, lstm.bias_hh_l0])
    y, hn, cn = r.forward(x.cuda(), h0.cuda(), c0.cuda())
    torch.cuda.synchronize()
    err = float((y.cpu() - y_ref).abs().max())
    r.close()
    if not err < 5e-2:
        raise RuntimeError(f"{name}: v1 forward differs from torch.nn.LSTM by {err}")
    return err


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="seq_len_sweep.md", help="where the table is written (markdown)")
    ap.add_argument("--lengths", default="64,192,448,960,1984,4032,8128")
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()
    lengths = [int(v) for v in a.lengths.split(",")]
    B, I, H = 32, 1024, 1024
    torch.manual_seed(0)
    lstm = torch.nn.LSTM(I, H)
    params = [lstm.weight_ih_l0, lstm.weight_hh_l0, lstm.bias_ih_l0, lstm.bias_hh_l0]
    libs = {}
    notes = []
    if os.path.exists(rg.REF_V1):
        libs["reference v1 (sm_100 rebuild)"] = rg.load(rg.REF_V1)
    else:
        notes.append("reference v1 library not built (python -m baseline.build_reference)")
    libs["this repository (v1 C ABI)"] = rg.load(rg.OURS)
    for name, lib in list(libs.items()):
        try:
            err = check_v1(lib, name, lstm, B, I, H)
            notes.append(f"{name}: max-abs error vs fp32 CPU torch.nn.LSTM on T=16: {err:.2e}")
        except Exception as exc:
            notes.append(f"{name}: NOT TIMED, {exc}")
            del libs[name]
    cud = torch.nn.LSTM(I, H).cuda().half()
    with torch.no_grad():
        for n, p in lstm.named_parameters():
            getattr(cud, n).copy_(p)
    rows = []
    for T in lengths:
        x = torch.randn(T, B, I, device="cuda")
        h0, c0 = torch.zeros(B, H, device="cuda"), torch.zeros(B, H, device="cuda")
        row = {"T": T}
        for name, lib in libs.items():
            for chunk in ((64, 0) if name.startswith("reference") else (0,)):
                try:
                    r = rg.V1Runner(lib, T, B, I, H, params, chunk=chunk)
                    sec = rg.time_calls(lambda: r.forward(x, h0, c0), a.warmup, a.iters)
                    r.close()
                    row[f"{name}, chunk {chunk}" if name.startswith("reference") else name] = sec * 1e3
                except Exception as exc:
                    row[f"{name}, chunk {chunk}"] = f"failed: {exc}"
        xh, h0h, c0h = x.half(), h0.half().unsqueeze(0), c0.half().unsqueeze(0)
        with torch.no_grad():
            sec = rg.time_calls(lambda: cud(xh, (h0h, c0h)), a.warmup, a.iters)
        row["torch.nn.LSTM fp16 (cuDNN)"] = sec * 1e3
        rows.append(row)
        print(json.dumps(row), flush=True)

    # input_proj_chunk_size sweep at T=2048 (what src/tune_projchunksz.cu:56-225 does: chunk in {0, 8, ..., 1024},
    # 1 warm-up + 5 timed), both libraries through the same calls
    chunk_rows = []
    Tc = 2048
    xc = torch.randn(Tc, B, I, device="cuda")
    h0c, c0c = torch.zeros(B, H, device="cuda"), torch.zeros(B, H, device="cuda")
    for chunk in (0, 8, 16, 32, 64, 128, 256, 512, 1024):
        row = {"chunk": chunk}
        for name, lib in libs.items():
            try:
                r = rg.V1Runner(lib, Tc, B, I, H, params, chunk=chunk)
                row[name] = rg.time_calls(lambda: r.forward(xc, h0c, c0c), 1, 5) * 1e3
                r.close()
            except Exception as exc:
                row[name] = f"failed: {exc}"
        chunk_rows.append(row)
        print(json.dumps(row), flush=True)

    # v2: forward + backward at benchmark configuration 2 through both libraries
    v2 = {}
    T2, B2, R = 512, 64, 1
    torch.manual_seed(1)
    x2, dy2 = torch.randn(T2, B2, I), torch.randn(T2, B2, H)
    h02, c02 = torch.randn(B2, H) * 0.1, torch.randn(B2, H) * 0.1
    v2libs = {"this repository (v2 C ABI)": rg.load(rg.OURS)}
    if os.path.exists(rg.REF_V2):
        v2libs["reference v2 (sm_100 rebuild)"] = rg.load(rg.REF_V2)
    else:
        notes.append("reference v2 library not built")
    with torch.no_grad():
        y_ref, _ = lstm(x2[:8].half().float(), (h02.half().float().unsqueeze(0), c02.half().float().unsqueeze(0)))
    for name, lib in v2libs.items():
        try:
            r = rg.V2Runner(lib, T2, B2, I, H, R, params, x2, h02, c02, dy2)
            r.forward()
            torch.cuda.synchronize()
            err = float((r.y[:8].float() - y_ref).abs().max())
            if not err < 5e-2:
                raise RuntimeError(f"forward differs from torch.nn.LSTM by {err}")

            def step():
                r.forward()
                r.backward()

            sec = rg.time_calls(step, a.warmup, a.iters)
            finite = bool(torch.isfinite(r.dx.float()).all()) and all(bool(torch.isfinite(g).all()) for g in r.G)
            v2[name] = {"ms_per_step": sec * 1e3, "tokens_per_s": T2 * B2 / sec, "y_max_abs_err_first_8_steps": err,
                        "gradients_finite": finite}
        except Exception as exc:
            v2[name] = {"failed": str(exc)[:300]}
        print(json.dumps({name: v2[name]}), flush=True)

    os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
    cols = [c for c in rows[0] if c != "T"] if rows else []
    with open(a.out, "w") as f:
        f.write("# Sequence-length sweep: B=32, I=H=1024, forward only (ms per call, median of %d)\n\n" % a.iters)
        f.write("Command: `python -m baseline.seq_len_sweep`\n\n")
        f.write("| T | " + " | ".join(cols) + " |\n|---|" + "---|" * len(cols) + "\n")
        for row in rows:
            f.write(f"| {row['T']} | " + " | ".join(
                (f"{row[c]:.3f}" if isinstance(row.get(c), float) else str(row.get(c, ""))) for c in cols) + " |\n")
        f.write("\n## input_proj_chunk_size sweep, T=2048, B=32, I=H=1024 (ms per call, median of 5)\n\n")
        ccols = [c for c in chunk_rows[0] if c != "chunk"] if chunk_rows else []
        f.write("| chunk | " + " | ".join(ccols) + " |\n|---|" + "---|" * len(ccols) + "\n")
        for row in chunk_rows:
            f.write(f"| {row['chunk']} | " + " | ".join(
                (f"{row[c]:.3f}" if isinstance(row.get(c), float) else str(row.get(c, ""))) for c in ccols) + " |\n")
        f.write("\n## v2 entry points, forward + backward, FP16, B=64, I=H=1024, T=512, R=1 (pinned host tensors)\n\n")
        for name, r in v2.items():
            f.write(f"* {name}: {json.dumps(r)}\n")
        f.write("\n## Notes\n\n" + "\n".join(f"* {n}" for n in notes) + "\n")
    print("wrote", a.out)


if __name__ == "__main__":
    main()
