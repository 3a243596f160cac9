"""The CPU oracle is pinned before anything is compared with it:
(1) against golden vectors produced by running the reference's own playground code
    (tests/golden/make_golden.py), and (2) against torch.nn.LSTM forward + autograd."""
import numpy as np
import pytest
import torch

from flashlstm_poc_b200.workloads import WORKLOADS, Inputs, make_inputs
from oracle import lstm_oracle as orc
from tests.helpers import golden_cases, params_from_inputs, torch_lstm_reference

ATOL, RTOL = 1e-5, 1e-5  # playground's own self-check uses atol 1e-5 (simple_lstm_bwd.py:305)


@pytest.mark.parametrize("path", golden_cases(), ids=lambda p: p.split("/")[-1][:-4])
def test_oracle_matches_reference_golden(path):
    g = np.load(path)
    params = [orc.LayerParams(g["w_ih"], g["w_hh"], g["b_ih"], g["b_hh"])]
    fwd = orc.lstm_forward(g["x"], params, g["h0"], g["c0"])
    np.testing.assert_allclose(fwd.y, g["y"], atol=ATOL, rtol=RTOL)
    np.testing.assert_allclose(fwd.h_n, g["hn"], atol=ATOL, rtol=RTOL)
    np.testing.assert_allclose(fwd.c_n, g["cn"], atol=ATOL, rtol=RTOL)
    np.testing.assert_allclose(fwd.caches[0].h_s, g["h_s"], atol=ATOL, rtol=RTOL)
    np.testing.assert_allclose(fwd.caches[0].c_s, g["c_s"], atol=ATOL, rtol=RTOL)
    np.testing.assert_allclose(fwd.caches[0].gates, g["gates"], atol=ATOL, rtol=RTOL)
    bwd = orc.lstm_backward(fwd, params, g["dy"], g["dhn"], g["dcn"])
    for name, got in (
        ("dx", bwd.dx), ("dh0", bwd.dh0[0]), ("dc0", bwd.dc0[0]), ("dw_ih", bwd.dw_ih[0]),
        ("dw_hh", bwd.dw_hh[0]), ("db_ih", bwd.db_ih[0]), ("db_hh", bwd.db_hh[0]),
    ):
        np.testing.assert_allclose(got, g[name], atol=2e-5, rtol=1e-4, err_msg=name)


@pytest.mark.parametrize("L,T,B,I,H", [(1, 7, 3, 5, 6), (2, 9, 4, 12, 8), (3, 4, 2, 6, 6), (1, 1, 1, 1, 1)])
def test_oracle_matches_torch_lstm(L, T, B, I, H):
    torch.manual_seed(100 + L + T)
    m = torch.nn.LSTM(I, H, num_layers=L)
    inp = Inputs(
        [getattr(m, f"weight_ih_l{l}").detach().clone() for l in range(L)],
        [getattr(m, f"weight_hh_l{l}").detach().clone() for l in range(L)],
        [getattr(m, f"bias_ih_l{l}").detach().clone() for l in range(L)],
        [getattr(m, f"bias_hh_l{l}").detach().clone() for l in range(L)],
        torch.randn(T, B, I), torch.randn(L, B, H), torch.randn(L, B, H), torch.randn(T, B, H),
    )
    dhn, dcn = torch.randn(L, B, H), torch.randn(L, B, H)
    ref = torch_lstm_reference(inp, dhn, dcn, dtype=torch.float64)
    params = params_from_inputs(inp)
    fwd = orc.lstm_forward(inp.x.numpy(), params, inp.h0.numpy(), inp.c0.numpy(), dtype=np.float64)
    bwd = orc.lstm_backward(fwd, params, inp.dy.numpy(), dhn.numpy(), dcn.numpy(), dtype=np.float64)
    tol = dict(atol=1e-9, rtol=1e-7)
    np.testing.assert_allclose(fwd.y, ref["y"], **tol)
    np.testing.assert_allclose(fwd.h_n, ref["hn"], **tol)
    np.testing.assert_allclose(fwd.c_n, ref["cn"], **tol)
    np.testing.assert_allclose(bwd.dx, ref["dx"], **tol)
    np.testing.assert_allclose(bwd.dh0, ref["dh0"], **tol)
    np.testing.assert_allclose(bwd.dc0, ref["dc0"], **tol)
    for l in range(L):
        np.testing.assert_allclose(bwd.dw_ih[l], ref["dw_ih"][l], **tol)
        np.testing.assert_allclose(bwd.dw_hh[l], ref["dw_hh"][l], **tol)
        np.testing.assert_allclose(bwd.db_ih[l], ref["db_ih"][l], **tol)
        np.testing.assert_allclose(bwd.db_hh[l], ref["db_hh"][l], **tol)


def test_oracle_config1_within_stated_tolerance():
    """Config 1 (fp32, I=H=256, B=32, T=128) at full size: fp32 oracle vs fp32 torch.nn.LSTM;
    tolerance = the bar the engine is held to (max-abs <= 2e-3)."""
    w = WORKLOADS["c1_fp32_h256"]
    inp = make_inputs(w)
    ref = torch_lstm_reference(inp)
    params = params_from_inputs(inp)
    fwd = orc.lstm_forward(inp.x.numpy(), params)
    bwd = orc.lstm_backward(fwd, params, inp.dy.numpy())
    assert orc.max_abs_err(fwd.y, ref["y"]) < 1e-4
    assert orc.max_abs_err(bwd.dx, ref["dx"]) < 2e-3
    assert orc.max_abs_err(bwd.dw_ih[0], ref["dw_ih"][0]) < 2e-3
    assert orc.max_abs_err(bwd.dw_hh[0], ref["dw_hh"][0]) < 2e-3
    assert orc.max_abs_err(bwd.db_ih[0], ref["db_ih"][0]) < 2e-3


def test_checkpoint_semantics():
    """Entry k of the h/c checkpoint tensors is the state entering step k*R; entry 0 = (h0, c0)."""
    g = np.load(golden_cases()[0])
    params = [orc.LayerParams(g["w_ih"], g["w_hh"], g["b_ih"], g["b_hh"])]
    fwd = orc.lstm_forward(g["x"], params, g["h0"], g["c0"])
    T = g["x"].shape[0]
    for R in (1, 2, 3, T, T + 5):
        ch, cc = orc.checkpoints(fwd.caches[0], R)
        assert ch.shape[0] == (T + R - 1) // R
        np.testing.assert_array_equal(ch[0], np.asarray(g["h0"][0], np.float32))
        np.testing.assert_array_equal(cc[0], np.asarray(g["c0"][0], np.float32))
        for k in range(ch.shape[0]):
            np.testing.assert_array_equal(ch[k], fwd.caches[0].h_s[k * R])


def test_workload_inputs_are_representable():
    w = WORKLOADS["c2_fp16_h1024"].scaled(seq_len=4, batch=2, input_size=32, hidden_size=32)
    inp = make_inputs(w)
    assert torch.equal(inp.x, inp.x.half().float())
    assert torch.equal(inp.w_hh[0], inp.w_hh[0].half().float())
    assert inp.h0 is not None and float(inp.h0.std()) < 0.2
