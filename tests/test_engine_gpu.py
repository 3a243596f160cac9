"""Parity of the CUDA engine (through the C ABI) with the CPU oracle, the reference-derived golden
vectors and torch.nn.LSTM.  Tolerances are the stated bar: max-abs <= 2e-3 for fp32, relative
L2 <= 1e-2 for FP16/BF16, against fp32 CPU ground truth computed on the same (rounded) inputs."""
import numpy as np
import pytest
import torch

from flashlstm_poc_b200.workloads import WORKLOADS, Inputs, Workload, make_inputs
from oracle import lstm_oracle as orc
from tests.gpu_helpers import assert_parity, run_engine, run_oracle
from tests.helpers import golden_cases, torch_lstm_reference

pytestmark = pytest.mark.gpu

BACKENDS = ["simt", "auto"]


@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: p.split("/")[-1][:-4])
def test_fp32_engine_matches_reference_golden(path):
    """The golden vectors come from running the reference's own CPU code; shapes include odd sizes
    (H=5, I=3) that no tile divides."""
    g = np.load(path)
    T, B, I = g["x"].shape
    H = g["w_hh"].shape[1]
    w = Workload("golden", "f32", 1, I, H, B, T, seed=0)
    t = lambda k: torch.from_numpy(g[k])
    inp = Inputs([t("w_ih")], [t("w_hh")], [t("b_ih")], [t("b_hh")], t("x"), t("h0"), t("c0"), t("dy"))
    got, eng = run_engine(w, inp, dhn=t("dhn"), dcn=t("dcn"))
    ref = {"y": g["y"], "hn": g["hn"], "cn": g["cn"], "dx": g["dx"], "dh0": g["dh0"], "dc0": g["dc0"],
           "dw_ih": [g["dw_ih"]], "dw_hh": [g["dw_hh"]], "db": [g["db_ih"]]}
    assert_parity(got, ref, "f32", fp32_max_abs=1e-4)
    gates = eng.gate_cache(0, T).float().cpu().numpy()
    assert orc.max_abs_err(gates, g["gates"]) < 1e-5
    eng.close()


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("L,T,B,I,H", [(1, 12, 8, 64, 64), (2, 9, 16, 128, 64), (1, 5, 3, 7, 6), (3, 4, 8, 64, 128)])
def test_engine_matches_oracle(backend, dtype, L, T, B, I, H):
    w = Workload("t", dtype, L, I, H, B, T, seed=11, state_std=0.5)
    inp = make_inputs(w)
    torch.manual_seed(5)
    rnd = lambda: torch.randn(L, B, H).to({"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dtype]).float()
    dhn, dcn = rnd(), rnd()
    got, eng = run_engine(w, inp, backend=backend, dhn=dhn, dcn=dcn)
    ref = run_oracle(inp, dhn, dcn)
    assert_parity(got, ref, dtype)
    eng.close()


def test_config1_fp32_full_size_against_torch_lstm():
    """Benchmark configuration 1 (fp32, I=H=256, B=32, T=128) at full size, ground truth = fp32 CPU torch.nn.LSTM (loss = sum(y*dY))."""
    w = WORKLOADS["c1_fp32_h256"]
    inp = make_inputs(w)
    got, eng = run_engine(w, inp)
    ref = torch_lstm_reference(inp)
    ref["db"] = ref["db_ih"]
    assert_parity(got, ref, "f32")
    eng.close()


@pytest.mark.parametrize("name,scale", [("c2_fp16_h1024", dict(seq_len=64, batch=64)),
                                        ("c3_bf16_l2_h2048", dict(seq_len=32, batch=32, input_size=512, hidden_size=512)),
                                        ("c5_bf16_l4_h1024", dict(seq_len=16, batch=64, input_size=256, hidden_size=256))])
def test_scaled_baseline_configs(name, scale):
    """The 16-bit benchmark configurations at sizes the CPU oracle finishes in seconds."""
    w = WORKLOADS[name].scaled(**scale)
    inp = make_inputs(w)
    got, eng = run_engine(w, inp)
    ref = run_oracle(inp)
    assert_parity(got, ref, w.dtype)
    eng.close()


@pytest.mark.parametrize("dtype,L,T,B,I,H,training,path", [
    ("bf16", 2, 5, 32, 2048, 2048, True, "auto"),    # config 3's width: W_hh slices do not fit shared memory -> streamed from L2
    ("f16", 1, 4, 8, 4096, 4096, False, "auto"),     # config 4: two row tiles per CTA, streamed weights, inference
    ("f16", 1, 3, 1, 4096, 4096, False, "auto"),     # config 4 at batch 1
    ("bf16", 2, 4, 256, 256, 1024, True, "auto"),    # 256 sequences at H=1024: two batch groups, one 128-wide tile each
    ("f16", 1, 5, 160, 128, 1024, True, "auto"),     # 128-wide tiles, the second one ragged (32 of 128 sequences)
    ("bf16", 1, 4, 192, 64, 512, False, "auto"),     # 128-wide tiles, inference, H=512
    ("bf16", 2, 4, 512, 256, 1024, True, "auto"),    # wide batch (config 5's regime): one GEMM launch per step, no K split
    ("bf16", 1, 4, 96, 128, 1024, True, "auto"),     # 96 sequences at H=1024: per-step path, one ragged 128-row tile
    ("bf16", 1, 3, 64, 256, 2048, True, "auto"),     # two batch tiles per CTA at H=2048: the planner takes the per-step path
    ("f16", 1, 5, 300, 128, 256, True, "step"),      # per-step path, ragged last 128-row tile, backward K split 8 ways
    ("bf16", 1, 3, 256, 128, 512, False, "step"),    # per-step path, inference
    ("f16", 1, 4, 40, 128, 128, True, "step"),       # per-step path with a single, mostly empty 128-row tile
    ("f16", 1, 6, 200, 192, 192, True, "auto"),      # ragged batch tile, K chunks not a multiple of 4
    ("bf16", 2, 4, 320, 256, 1024, True, "persistent"),  # the persistent kernels with several batch tiles per CTA: five
                                                         # 64-wide tiles over two batch groups, one slot without sequences
    ("f16", 1, 4, 96, 128, 2048, True, "persistent"),    # streamed weights with three 32-wide tiles per CTA
])
def test_wide_and_large_batch_regimes(dtype, L, T, B, I, H, training, path, monkeypatch):
    if path == "persistent":
        monkeypatch.setenv("FLSTM_STEP_MIN_BATCH", "0")  # keep wide batches on the persistent kernels
    elif path == "step":
        monkeypatch.setenv("FLSTM_STEP_MIN_BATCH", "1")  # per-step GEMM launches whatever the planner would pick
    w = Workload("t", dtype, L, I, H, B, T, seed=17, state_std=0.2, training=training)
    inp = make_inputs(w)
    got, eng = run_engine(w, inp, backend="tc")
    ref = run_oracle(inp)
    assert_parity(got, ref, dtype)
    eng.close()


def test_weight_gradient_gemms_side_by_side(monkeypatch):
    """FLSTM_DW_SIDE_BY_SIDE=1: dW_ih and dW_hh of a layer are computed at the same time on two streams, each GEMM on
    its share of the SMs; same results as one after the other."""
    monkeypatch.setenv("FLSTM_DW_SIDE_BY_SIDE", "1")
    w = Workload("t", "bf16", 2, 256, 256, 32, 6, seed=5, state_std=0.2)
    inp = make_inputs(w)
    got, eng = run_engine(w, inp, backend="tc", repeat=2)
    assert_parity(got, run_oracle(inp), "bf16")
    eng.close()


def test_repeatable_and_cache_layout():
    """Two runs give bit-identical results (a race in a persistent kernel's barrier would not), and
    the gate cache read back in torch order matches the oracle's activations."""
    w = Workload("t", "f16", 1, 64, 64, 16, 10, seed=3, state_std=0.3)
    inp = make_inputs(w)
    a, eng = run_engine(w, inp)
    b, eng2 = run_engine(w, inp, repeat=2)
    for k in ("y", "dx", "dh0"):
        assert np.array_equal(a[k], b[k]), k
    assert np.array_equal(a["dw_hh"][0], b["dw_hh"][0])
    ref = run_oracle(inp)
    gates = eng.gate_cache(0, w.seq_len).float().cpu().numpy()
    assert orc.max_abs_err(gates, ref["gates"][0]) < 5e-3
    eng.close(); eng2.close()


def test_sequence_length_may_change_between_calls():
    """The v1 contract: T differs per call and the workspace grows (src/lstm.cu:933-970)."""
    w = Workload("t", "f16", 1, 32, 32, 4, 6, seed=9)
    base = make_inputs(w)
    dev = torch.device("cuda", 0)
    from flashlstm_poc_b200.engine import Engine

    eng = Engine("f16", 1, 4, 32, 32, max_seq_len=6, training=False, device=dev)
    eng.set_weights(0, base.w_ih[0].to(dev), base.w_hh[0].to(dev), base.b_ih[0].to(dev), base.b_hh[0].to(dev))
    for T in (6, 3, 13):
        ww = w.scaled(seq_len=T, training=False)
        inp = make_inputs(ww)
        inp.w_ih, inp.w_hh, inp.b_ih, inp.b_hh = base.w_ih, base.w_hh, base.b_ih, base.b_hh
        y, hn, cn = eng.forward(inp.x.to(dev, torch.float16))
        ref = run_oracle(inp)
        assert orc.rel_l2_err(y.float().cpu().numpy(), ref["y"]) < 1e-2
    eng.close()


def test_errors_are_reported():
    from flashlstm_poc_b200._lib import FlashLstmError
    from flashlstm_poc_b200.engine import Engine

    dev = torch.device("cuda", 0)
    eng = Engine("f16", 1, 2, 8, 8, 4, device=dev)
    x = torch.zeros(4, 2, 8, dtype=torch.float16, device=dev)
    with pytest.raises(FlashLstmError, match="weights"):
        eng.forward(x)
    with pytest.raises(ValueError):
        eng.forward(x.float())
    with pytest.raises(FlashLstmError):
        Engine("f32", 1, 2, 8, 8, 4, backend="tc", device=dev)  # tensor-core path is 16-bit only
    eng.close()


@pytest.mark.parametrize("dtype,L,H", [("f16", 1, 128), ("bf16", 2, 64), ("f32", 1, 32)])
def test_whole_step_in_a_cuda_graph(dtype, L, H):
    """Forward + backward captured once and replayed on new inputs gives what the eager calls give."""
    from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine

    dev = torch.device("cuda", 0)
    td = TORCH_DTYPES[dtype]
    T, B, I = 9, 16, 64
    w = Workload("g", dtype, L, I, H, B, T, seed=31, state_std=0.2)
    inp = make_inputs(w)
    eng = Engine(dtype, L, B, I, H, T, device=dev)
    for l in range(L):
        eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
    x = torch.zeros(T, B, I, dtype=td, device=dev)
    dy = torch.zeros(T, B, H, dtype=td, device=dev)
    h0, c0 = inp.h0.to(dev, td), inp.c0.to(dev, td)
    y = torch.empty(T, B, H, dtype=td, device=dev)
    hn, cn = torch.empty(L, B, H, dtype=td, device=dev), torch.empty(L, B, H, dtype=td, device=dev)
    dx = torch.empty(T, B, I, dtype=td, device=dev)
    dh0, dc0 = torch.empty(L, B, H, device=dev), torch.empty(L, B, H, device=dev)
    graph = eng.capture_step(x, h0, c0, y, hn, cn, dy, dx, dh0, dc0)
    x.copy_(inp.x.to(dev, td))
    dy.copy_(inp.dy.to(dev, td))
    graph.replay()
    torch.cuda.synchronize()
    got = {"y": y.float().cpu().numpy(), "dx": dx.float().cpu().numpy(), "dh0": dh0.cpu().numpy(),
           "dw_hh": [eng.grads(l)[1].cpu().numpy() for l in range(L)]}
    ref = run_oracle(inp)
    assert_parity(got, ref, dtype, keys=["y", "dx", "dh0", "dw_hh"])
    y1 = y.clone()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, y1)
    eng.close()


@pytest.mark.parametrize("dtype,L,H,backend", [("f16", 1, 128, "tc"), ("bf16", 2, 64, "tc"), ("f32", 2, 24, "simt"),
                                               ("f16", 1, 1024, "tc")])
def test_step_ranges_equal_one_call(dtype, L, H, backend, B=16):
    """A sequence run as ascending forward ranges and descending backward ranges gives bit-identical
    results to the single forward / backward calls (the ranges are what host streaming pipelines)."""
    from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine

    dev = torch.device("cuda", 0)
    td = TORCH_DTYPES[dtype]
    T, I = 23, 64
    w = Workload("r", dtype, L, I, H, B, T, seed=41, state_std=0.2)
    inp = make_inputs(w)
    torch.manual_seed(3)
    dhn = torch.randn(L, B, H).to(td).to(dev)
    dcn = torch.randn(L, B, H).to(td).to(dev)

    def run(cuts):
        eng = Engine(dtype, L, B, I, H, T, device=dev, backend=backend)
        for l in range(L):
            eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
        x, dy = inp.x.to(dev, td), inp.dy.to(dev, td)
        h0, c0 = inp.h0.to(dev, td), inp.c0.to(dev, td)
        y = torch.zeros(T, B, H, dtype=td, device=dev)
        hn, cn = torch.zeros(L, B, H, dtype=td, device=dev), torch.zeros(L, B, H, dtype=td, device=dev)
        dx = torch.zeros(T, B, I, dtype=td, device=dev)
        dh0, dc0 = torch.zeros(L, B, H, device=dev), torch.zeros(L, B, H, device=dev)
        edges = [0] + cuts + [T]
        for a, b in zip(edges[:-1], edges[1:]):
            eng.forward_range_into(T, a, b, x, h0, c0, y, hn, cn)
        for a, b in reversed(list(zip(edges[:-1], edges[1:]))):
            eng.backward_range_into(T, a, b, dy, dhn, dcn, dx, dh0, dc0)
        torch.cuda.synchronize()
        out = [y, hn, cn, dx, dh0, dc0] + [g.clone() for l in range(L) for g in eng.grads(l)]
        out = [o.clone() for o in out]
        eng.close()
        return out

    whole = run([])
    for cuts in ([8, 16], [1, 2, 22], [11]):
        parts = run(cuts)
        for a, b in zip(whole, parts):
            assert torch.equal(a, b), cuts
    ref = run_oracle(inp, dhn.float().cpu(), dcn.float().cpu())
    got = {"y": whole[0].float().cpu().numpy(), "dx": whole[3].float().cpu().numpy(), "dh0": whole[4].cpu().numpy()}
    assert_parity(got, ref, dtype, keys=["y", "dx", "dh0"])


def test_step_ranges_wide_batch():
    """The same for the wide-batch path, whose fp32 partial sums of dh carry over between ranges."""
    import os

    os.environ["FLSTM_STEP_MIN_BATCH"] = "1"
    try:
        test_step_ranges_equal_one_call("bf16", 2, 128, "tc", B=256)
    finally:
        del os.environ["FLSTM_STEP_MIN_BATCH"]


@pytest.mark.parametrize("dtype,L,T,B,I,H,chunk", [("bf16", 3, 7, 256, 128, 256, 2), ("f16", 2, 9, 300, 256, 128, 4),
                                                   ("bf16", 4, 6, 256, 128, 128, 1)])
def test_cross_layer_wavefront(dtype, L, T, B, I, H, chunk, monkeypatch):
    """Stacked layers on the per-step path run as a wavefront (layer l on time chunk k while layer l-1 is on
    chunk k+1, one stream per layer).  Same kernels in the same per-layer order, so the results are
    bit-identical to the layer-by-layer schedule, and they match the oracle."""
    monkeypatch.setenv("FLSTM_STEP_MIN_BATCH", "1")
    w = Workload("t", dtype, L, I, H, B, T, seed=23, state_std=0.2)
    inp = make_inputs(w)
    monkeypatch.setenv("FLSTM_WAVE_CHUNK", str(chunk))
    wave, eng = run_engine(w, inp, backend="tc")
    eng.close()
    monkeypatch.setenv("FLSTM_WAVE_CHUNK", "0")
    flat, eng = run_engine(w, inp, backend="tc")
    eng.close()
    for k in wave:
        a, b = wave[k], flat[k]
        if isinstance(a, list):
            assert all(np.array_equal(x, y) for x, y in zip(a, b)), k
        else:
            assert np.array_equal(a, b), k
    assert_parity(wave, run_oracle(inp), dtype)


def test_host_watchdog_wait():
    """flstm_engine_wait: a deadline that cannot be met is reported as TIMEOUT without disturbing the work in
    flight (nothing is cancelled on the GPU; only an attached communicator would be aborted); a generous one
    returns once the step is done, and the results are the same as without any waiting."""
    from flashlstm_poc_b200._lib import FlashLstmError
    from flashlstm_poc_b200.engine import Engine

    dev = torch.device("cuda", 0)
    w = WORKLOADS["c2_fp16_h1024"].scaled(seq_len=256)
    inp = make_inputs(w)
    eng = Engine("f16", 1, w.batch, w.input_size, w.hidden_size, w.seq_len, device=dev)
    eng.set_weights(0, inp.w_ih[0].to(dev), inp.w_hh[0].to(dev), inp.b_ih[0].to(dev), inp.b_hh[0].to(dev))
    x, dy = inp.x.to(dev, torch.float16), inp.dy.to(dev, torch.float16)
    y0, _, _ = eng.forward(x)
    eng.backward(dy)
    torch.cuda.synchronize()
    y0 = y0.clone()
    y1, _, _ = eng.forward(x)   # a few milliseconds of device work, enqueued asynchronously
    eng.backward(dy)
    with pytest.raises(FlashLstmError, match="did not finish within 0 ms"):
        eng.wait(0.0)
    eng.wait(30.0)              # returns as soon as the step is done
    assert torch.cuda.current_stream().query()
    assert torch.equal(y0, y1)
    eng.abort_comm()            # no communicator attached: a no-op
    eng.forward(x)
    eng.wait(30.0)
    eng.close()


def test_step_ranges_must_be_in_order():
    from flashlstm_poc_b200._lib import FlashLstmError
    from flashlstm_poc_b200.engine import Engine

    dev = torch.device("cuda", 0)
    w = Workload("r", "f16", 1, 64, 64, 8, 8, seed=1)
    inp = make_inputs(w)
    eng = Engine("f16", 1, 8, 64, 64, 8, device=dev)
    eng.set_weights(0, inp.w_ih[0].to(dev), inp.w_hh[0].to(dev), inp.b_ih[0].to(dev), inp.b_hh[0].to(dev))
    x = inp.x.to(dev, torch.float16)
    y = torch.empty(8, 8, 64, dtype=torch.float16, device=dev)
    eng.forward_range_into(8, 0, 4, x, None, None, y, None, None)
    with pytest.raises(FlashLstmError, match="contiguous"):
        eng.forward_range_into(8, 5, 8, x, None, None, y, None, None)
    with pytest.raises(FlashLstmError, match="does not follow"):
        eng.backward_range_into(8, 4, 8, y, None, None, None, None, None)  # the forward is not complete yet
    eng.forward_range_into(8, 4, 8, x, None, None, y, None, None)
    with pytest.raises(FlashLstmError, match="descending"):
        eng.backward_range_into(8, 0, 4, y, None, None, None, None, None)
    eng.close()


def test_step_trace_of_the_persistent_kernels_is_ordered():
    """The in-kernel step trace (flstm_engine_enable_trace): every step's stamps ascend from the barrier to the
    release, in the forward and in the BPTT kernel."""
    from flashlstm_poc_b200 import step_trace
    from flashlstm_poc_b200.engine import Engine

    w = Workload("trace", "f16", 1, 256, 256, 32, 24, seed=2)
    inp = make_inputs(w)
    dev = torch.device("cuda", 0)
    eng = Engine(w.dtype, 1, w.batch, w.input_size, w.hidden_size, w.seq_len, device=dev)
    eng.set_weights(0, inp.w_ih[0].to(dev), inp.w_hh[0].to(dev), inp.b_ih[0].to(dev), inp.b_hh[0].to(dev))
    x, dy = inp.x.to(dev, torch.float16), inp.dy.to(dev, torch.float16)

    def run_step():
        eng.forward(x)
        eng.backward(dy)

    run_step()
    stamps = step_trace.collect(eng, run_step, steps=16)
    summary = step_trace.summarize(stamps, skip=2)
    eng.close()
    for kernel in ("forward", "bptt"):
        rows = summary[kernel]
        assert rows["period"] > 0
        assert 0 < rows["step barrier satisfied"] < rows["last UMMA committed"] < rows["released"] <= rows["period"] * 1.5
