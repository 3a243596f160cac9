"""Host streaming with a bounded device footprint.

The reference keeps 2 x 32 steps of a sequence on the GPU and the rest in pinned host memory, and its backward
recomputes from h/c checkpoints (flashlstm_v2/src/lstm_forward.cu:515,673-940, lstm_backward.cu:496-523,975-1054).
Here: (1) the native building blocks -- a segment-sized engine fed segment by segment, flstm_engine_backward_segment
consuming caller-held checkpoints; (2) the reference's v2 C ABI with a device-memory cap so small that the
sequence cannot stay resident: the shim streams it in segments, the backward consumes the caller's checkpoint
tensors, and the device footprint does not depend on T."""
import ctypes
import os

import numpy as np
import pytest
import torch

from flashlstm_poc_b200 import _lib
from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine
from flashlstm_poc_b200.workloads import Workload, make_inputs
from oracle import lstm_oracle as orc
from tests.gpu_helpers import assert_parity, run_oracle
from tests.helpers import to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,layers,batch,hidden,T,S", [("bf16", 2, 16, 128, 80, 32), ("f16", 1, 96, 1024, 20, 8)])
def test_engine_streams_a_sequence_in_segments(dtype, layers, batch, hidden, T, S):
    """A T-step sequence through an engine whose workspace holds S steps: forward segment after segment with the
    states carried by the caller, backward from the last segment to the first with flstm_engine_backward_segment."""
    w = Workload("stream", dtype, layers, 128, hidden, batch, T, seed=21, state_std=0.2)
    inp = make_inputs(w)
    dev = torch.device("cuda", 0)
    td = TORCH_DTYPES[dtype]
    eng = Engine(dtype, layers, batch, w.input_size, hidden, S, device=dev)
    for l in range(layers):
        eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
    eng.set_recompute_interval(S)
    eng.set_cell_io_f32(True)
    workspace = eng.workspace_bytes
    x, dy = inp.x.to(dev, td), inp.dy.to(dev, td)
    h = inp.h0.to(dev, td)
    c = inp.c0.to(dev, td).float()  # the initial cell state as the 16-bit value the oracle sees
    y = torch.empty(T, batch, hidden, dtype=td, device=dev)
    bounds = [(a, min(a + S, T)) for a in range(0, T, S)]
    ck = []
    for a, b in bounds:  # forward, in time order; the states entering each segment are its checkpoint
        ck.append((h, c))
        hn = torch.empty_like(h)
        cn = torch.empty_like(c)
        eng.forward_into(b - a, x[a:b], h, c, y[a:b], hn, cn)
        h, c = hn, cn
    dx = torch.empty(T, batch, w.input_size, dtype=td, device=dev)
    dh0 = torch.empty(layers, batch, hidden, device=dev)
    dc0 = torch.empty(layers, batch, hidden, device=dev)
    for k in reversed(range(len(bounds))):  # backward, last segment first
        a, b = bounds[k]
        eng.backward_segment_into(b - a, k == len(bounds) - 1, k == 0, x[a:b], ck[k][0], ck[k][1], dy[a:b], None, None,
                                  dx[a:b], dh0, dc0)
    torch.cuda.synchronize()
    assert eng.workspace_bytes == workspace  # nothing grew with T
    got = dict(y=to_np(y), hn=to_np(h), cn=to_np(c), dx=to_np(dx), dh0=to_np(dh0), dc0=to_np(dc0))
    got["dw_ih"], got["dw_hh"], got["db"] = map(list, zip(*[[to_np(g) for g in eng.grads(l)] for l in range(layers)]))
    eng.close()
    assert_parity(got, run_oracle(inp), dtype)


def _v2_step(lib, T, B, I, H, R, lstm, x, h0, c0, dy, fresh_cache_for_backward):
    dev = "cuda"
    P = [p.detach().to(dev).contiguous() for p in (lstm.weight_ih_l0, lstm.weight_hh_l0, lstm.bias_ih_l0, lstm.bias_hh_l0)]
    nchk = (T + R - 1) // R
    y = torch.empty(T, B, H, dtype=torch.float16).pin_memory()
    ch = torch.empty(nchk, B, H, dtype=torch.float16).pin_memory()
    cc = torch.empty(nchk, B, H, dtype=torch.float32).pin_memory()
    h0d, c0d = h0.to(dev), c0.to(dev)
    hy, cy = torch.empty_like(h0d), torch.empty_like(c0d)
    streams = [torch.cuda.Stream() for _ in range(3)]
    opt = _lib.StreamingLstmOptions(1, 0)
    cache = _lib.GateCacheHost(ch.data_ptr(), cc.data_ptr())
    torch.cuda.synchronize()
    s = [st.cuda_stream for st in streams]
    lib.flstm_StreamingLstmForward(T, B, I, H, R, x.data_ptr(), h0d.data_ptr(), c0d.data_ptr(), P[0].data_ptr(), P[1].data_ptr(),
                                   P[2].data_ptr(), P[3].data_ptr(), y.data_ptr(), cache, ctypes.byref(opt), hy.data_ptr(),
                                   cy.data_ptr(), s[0], s[1], s[2])
    assert lib.flstm_last_status() == 0, lib.flstm_last_error()
    nbytes, streaming = ctypes.c_size_t(), ctypes.c_int()
    lib.flstm_v2_last_call_info(ctypes.byref(nbytes), ctypes.byref(streaming))
    dx = torch.empty(T, B, I, dtype=torch.float16).pin_memory()
    G = [torch.empty_like(p) for p in P]
    dh0, dc0 = torch.empty(B, H, device=dev), torch.empty(B, H, device=dev)
    lib.flstm_StreamingLstmBackward(T, B, I, H, R, x.data_ptr(), y.data_ptr(), cache, dy.data_ptr(), None, None, h0d.data_ptr(),
                                    c0d.data_ptr(), P[0].data_ptr(), P[1].data_ptr(), P[2].data_ptr(), P[3].data_ptr(),
                                    dx.data_ptr(), G[0].data_ptr(), G[1].data_ptr(), G[2].data_ptr(), G[3].data_ptr(),
                                    dh0.data_ptr(), dc0.data_ptr(), s[0], s[1], s[2], ctypes.byref(opt))
    assert lib.flstm_last_status() == 0, lib.flstm_last_error()
    out = dict(y=y.float().numpy(), hn=hy.float().cpu().numpy(), cn=cy.float().cpu().numpy(), dx=dx.float().numpy(),
               dh0=dh0.cpu().numpy(), dc0=dc0.cpu().numpy(), dw_ih=G[0].cpu().numpy(), dw_hh=G[1].cpu().numpy(),
               db=G[2].cpu().numpy(), ch=ch.float().numpy(), cc=cc.numpy())
    return out, nbytes.value, streaming.value


@pytest.mark.parametrize("R", [4, 32])
def test_v2_surface_streams_when_the_sequence_exceeds_the_device_budget(R, monkeypatch):
    """T*B*H far beyond a 4 MB device budget: the v2 shim must run in streaming mode, its backward must consume
    the caller's checkpoints, the results must match fp32 torch.nn.LSTM (relative L2 <= 1e-2), and the device
    footprint must be the same for T = 200 and T = 400."""
    lib = _lib.load()
    monkeypatch.setenv("FLSTM_V2_DEVICE_BUDGET_BYTES", str(4 << 20))
    B, I, H = 16, 128, 128
    torch.manual_seed(3)
    lstm = torch.nn.LSTM(I, H)
    footprints = []
    for T in (200, 400):
        x = torch.randn(T, B, I).half().pin_memory()
        dy = torch.randn(T, B, H).half().pin_memory()
        h0, c0 = (torch.randn(B, H) * 0.3).half(), (torch.randn(B, H) * 0.3).half()
        got, nbytes, streaming = _v2_step(lib, T, B, I, H, R, lstm, x, h0, c0, dy, True)
        assert streaming == 1
        footprints.append(nbytes)
        xr = x.float().requires_grad_(True)
        h0r, c0r = h0.float().unsqueeze(0).requires_grad_(True), c0.float().unsqueeze(0).requires_grad_(True)
        y_ref, (hn_ref, cn_ref) = lstm(xr, (h0r, c0r))
        lstm.zero_grad()
        (y_ref * dy.float()).sum().backward()
        ref = dict(y=y_ref, hn=hn_ref[0], cn=cn_ref[0], dx=xr.grad, dh0=h0r.grad[0], dc0=c0r.grad[0],
                   dw_ih=lstm.weight_ih_l0.grad, dw_hh=lstm.weight_hh_l0.grad, db=lstm.bias_ih_l0.grad)
        for k, v in ref.items():
            err = orc.rel_l2_err(got[k], v.detach().numpy())
            assert err < 1e-2, (T, k, err)
        # checkpoints: entry e = state entering step e*R; entry 0 = h0 / c0
        assert np.array_equal(got["ch"][0], h0.float().numpy())
        for e in range(1, (T + R - 1) // R):
            assert orc.rel_l2_err(got["ch"][e], y_ref[e * R - 1].detach().numpy()) < 1e-2
    assert footprints[0] == footprints[1] and 0 < footprints[0] <= (6 << 20)
