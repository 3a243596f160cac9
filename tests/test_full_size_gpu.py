"""The two large BF16 benchmark configurations at FULL size on the GPU, checked on a batch slice.

Sequences are independent across the batch in the forward pass and in dx / dh0 / dc0, so the CPU oracle is
run on a few rows of the batch only (seconds instead of minutes) and compared with the same rows of the
engine's full-size run.  Weight gradients sum over the batch; they are covered at reduced batch by the other
parity tests."""
import numpy as np
import pytest
import torch

from flashlstm_poc_b200.engine import Engine
from flashlstm_poc_b200.workloads import WORKLOADS, Inputs, make_inputs
from oracle import lstm_oracle as orc
from tests.gpu_helpers import run_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,rows", [("c3_bf16_l2_h2048", [0, 130, 255]), ("c5_bf16_l4_h1024", [0, 1, 700, 2047])])
def test_full_size_batch_slice_matches_oracle(name, rows):
    w = WORKLOADS[name]
    inp = make_inputs(w)
    dev = torch.device("cuda", 0)
    td = torch.bfloat16
    eng = Engine(w.dtype, w.layers, w.batch, w.input_size, w.hidden_size, w.seq_len, device=dev)
    for l in range(w.layers):
        eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
    x, dy = inp.x.to(dev, td), inp.dy.to(dev, td)
    y, hn, cn = eng.forward(x)
    dx, dh0, dc0 = eng.backward(dy)
    torch.cuda.synchronize()
    idx = torch.tensor(rows, device=dev)
    got = {"y": y.index_select(1, idx), "hn": hn.index_select(1, idx), "cn": cn.index_select(1, idx),
           "dx": dx.index_select(1, idx), "dh0": dh0.index_select(1, idx), "dc0": dc0.index_select(1, idx)}
    got = {k: v.float().cpu().numpy() for k, v in got.items()}
    finite = all(bool(torch.isfinite(t.float()).all()) for t in (y, dx, dh0, dc0))
    eng.close()
    del x, dy, y, dx
    assert finite
    sl = Inputs(inp.w_ih, inp.w_hh, inp.b_ih, inp.b_hh, inp.x[:, rows].contiguous(), None, None, inp.dy[:, rows].contiguous())
    ref = run_oracle(sl)
    for k, v in got.items():
        err = orc.rel_l2_err(v, ref[k])
        assert err < 1e-2, (k, err)   # the stated bar for 16-bit configurations: relative L2 <= 1e-2


def test_config2_full_size_all_outputs():
    """The benchmark configuration itself (FP16, I=H=1024, B=64, T=512), every output including the weight
    gradients, against the oracle on the whole batch."""
    from tests.gpu_helpers import assert_parity, run_engine

    w = WORKLOADS["c2_fp16_h1024"]
    inp = make_inputs(w)
    got, eng = run_engine(w, inp)
    assert eng.backend == "tc"
    eng.close()
    assert_parity(got, run_oracle(inp), w.dtype)


def test_config4_full_size_inference_slice():
    """Configuration 4 (FP16, I=H=4096, T=2048, B=8, forward only, W_hh streamed from HBM every step): two of
    the eight sequences against the oracle."""
    w = WORKLOADS["c4_fp16_h4096_b8"]
    inp = make_inputs(w)
    dev = torch.device("cuda", 0)
    eng = Engine(w.dtype, 1, w.batch, w.input_size, w.hidden_size, w.seq_len, training=False, device=dev)
    eng.set_weights(0, inp.w_ih[0].to(dev), inp.w_hh[0].to(dev), inp.b_ih[0].to(dev), inp.b_hh[0].to(dev))
    y, hn, cn = eng.forward(inp.x.to(dev, torch.float16))
    torch.cuda.synchronize()
    rows = [0, 7]
    got = {"y": y[:, rows].float().cpu().numpy(), "hn": hn[:, rows].float().cpu().numpy(), "cn": cn[:, rows].float().cpu().numpy()}
    eng.close()
    ref = run_oracle(Inputs(inp.w_ih, inp.w_hh, inp.b_ih, inp.b_hh, inp.x[:, rows].contiguous(), None, None, None))
    for k, v in got.items():
        err = orc.rel_l2_err(v, ref[k])
        assert err < 1e-2, (k, err)
