"""Activation checkpoints (recompute interval R): the forward keeps only the h/c state entering every R-th step,
the backward rebuilds the gate cache one segment at a time.  Outputs and state gradients must be bit-identical
to the full-cache engine (same kernels on the same values), weight gradients equal up to the fp32 order of the
segment-by-segment sum, everything within the parity bar against the CPU oracle, and the workspace smaller."""
import numpy as np
import pytest
import torch

from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine
from flashlstm_poc_b200.workloads import Workload, make_inputs
from tests.gpu_helpers import assert_parity, run_oracle
from tests.helpers import to_np

pytestmark = pytest.mark.gpu


def _run(w, inp, interval, dhn, dcn, repeat=1):
    dev = torch.device("cuda", 0)
    td = TORCH_DTYPES[w.dtype]
    eng = Engine(w.dtype, w.layers, w.batch, w.input_size, w.hidden_size, w.seq_len, device=dev, backend="tc")
    for l in range(w.layers):
        eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
    if interval:
        eng.set_recompute_interval(interval)
    out = {}
    x, h0, c0, dy = inp.x.to(dev, td), inp.h0.to(dev, td), inp.c0.to(dev, td), inp.dy.to(dev, td)  # x must outlive backward
    for _ in range(repeat):
        y, hn, cn = eng.forward(x, h0, c0)
        dx, dh0, dc0 = eng.backward(dy, dhn.to(dev, td), dcn.to(dev, td))
        out = dict(y=to_np(y), hn=to_np(hn), cn=to_np(cn), dx=to_np(dx), dh0=to_np(dh0), dc0=to_np(dc0),
                   dw_ih=[to_np(eng.grads(l)[0]) for l in range(w.layers)],
                   dw_hh=[to_np(eng.grads(l)[1]) for l in range(w.layers)],
                   db=[to_np(eng.grads(l)[2]) for l in range(w.layers)])
    torch.cuda.synchronize()
    bytes_ = eng.workspace_bytes
    eng.close()
    return out, bytes_


@pytest.mark.parametrize("dtype,L,T,B,I,H,R,step_path", [
    ("f16", 2, 23, 16, 64, 64, 5, False),     # persistent kernels, ragged last segment, stacked layers
    ("bf16", 1, 12, 32, 128, 128, 1, False),  # R = 1: a checkpoint at every step
    ("f16", 1, 9, 8, 64, 128, 16, False),     # R >= T: a single segment
    ("bf16", 2, 9, 256, 128, 128, 4, True),   # per-step GEMM path (wide batch), dh carried as fp32 partial sums
    ("f16", 1, 7, 300, 64, 256, 3, True),     # per-step path, ragged batch tile, K split
])
def test_checkpoint_mode_matches_full_cache(dtype, L, T, B, I, H, R, step_path, monkeypatch):
    monkeypatch.setenv("FLSTM_STEP_MIN_BATCH", "1" if step_path else "0")
    w = Workload("ck", dtype, L, I, H, B, T, seed=77, state_std=0.3)
    inp = make_inputs(w)
    torch.manual_seed(9)
    td = TORCH_DTYPES[dtype]
    dhn, dcn = torch.randn(L, B, H).to(td), torch.randn(L, B, H).to(td)
    full, full_bytes = _run(w, inp, 0, dhn, dcn)
    ck, ck_bytes = _run(w, inp, R, dhn, dcn, repeat=2)   # twice: the carries and accumulators start over
    for k in ("y", "hn", "cn", "dx", "dh0", "dc0"):
        assert np.array_equal(full[k], ck[k]), k
    for k in ("dw_ih", "dw_hh", "db"):
        for a, b in zip(full[k], ck[k]):
            assert np.linalg.norm(a - b) <= 1e-5 * np.linalg.norm(a) + 1e-7, k
    ref = run_oracle(inp, dhn.float(), dcn.float())
    assert_parity(ck, ref, dtype)
    if R < T:
        assert ck_bytes < full_bytes


def test_checkpoint_mode_limits():
    from flashlstm_poc_b200._lib import FlashLstmError

    dev = torch.device("cuda", 0)
    eng = Engine("f32", 1, 4, 16, 16, 8, device=dev)   # fp32 runs on the SIMT backend
    with pytest.raises(FlashLstmError, match="tensor-core backend"):
        eng.set_recompute_interval(4)
    eng.close()
    w = Workload("ck", "f16", 1, 64, 64, 8, 8, seed=1)
    inp = make_inputs(w)
    eng = Engine("f16", 1, 8, 64, 64, 8, device=dev)
    eng.set_weights(0, inp.w_ih[0].to(dev), inp.w_hh[0].to(dev), inp.b_ih[0].to(dev), inp.b_hh[0].to(dev))
    eng.set_recompute_interval(4)
    x = inp.x.to(dev, torch.float16)
    y = torch.empty(8, 8, 64, dtype=torch.float16, device=dev)
    with pytest.raises(FlashLstmError, match="step ranges"):
        eng.forward_range_into(8, 0, 4, x, None, None, y, None, None)
    eng.set_recompute_interval(0)   # back to the full gate cache
    eng.forward_range_into(8, 0, 4, x, None, None, y, None, None)
    eng.forward_range_into(8, 4, 8, x, None, None, y, None, None)
    torch.cuda.synchronize()
    eng.close()
