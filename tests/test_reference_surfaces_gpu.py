"""The reference's own tests for this path, re-stated against the drop-in surfaces:
  * v1 C ABI through ctypes            <- python/test_lstm.py:87-273 (presets :280-302)
  * StreamingLSTM module               <- flashlstm_v2/python/tests/test_streaming_lstm.py:14-89
  * v2 C ABI through ctypes            <- flashlstm_v2/scripts/validate_lstm_fwd.py:97-250,
                                          validate_lstm_bwd.py:283-443
Ground truth is CPU fp32 torch.nn.LSTM on the fp16-rounded inputs, as in those tests."""
import ctypes

import numpy as np
import pytest
import torch

from flashlstm_poc_b200 import _lib
from oracle import lstm_oracle as orc

pytestmark = pytest.mark.gpu

V1_PRESETS = [(1, 1, 4, 4), (3, 2, 8, 8), (5, 1, 16, 12), (8, 2, 32, 24), (16, 2, 64, 48), (32, 2, 128, 96),
              (7, 3, 24, 16), (24, 8, 64, 64)]


def _v1_forward(lib, bufs, lstm, x, h0, c0, T, B, I, H, prec):
    dev = "cuda"
    out = torch.empty(T * B * H, dtype=torch.float32, device=dev)
    hn = torch.empty(B * H, dtype=torch.float32, device=dev)
    cn = torch.empty(B * H, dtype=torch.float32, device=dev)
    xd, h0d, c0d = x.to(dev).contiguous(), h0.to(dev).contiguous(), c0.to(dev).contiguous()
    bi, bh = lstm.bias_ih_l0.detach().to(dev), lstm.bias_hh_l0.detach().to(dev)
    st = lib.lstm_forward(xd.data_ptr(), bi.data_ptr(), bh.data_ptr(), h0d.data_ptr(), c0d.data_ptr(), out.data_ptr(),
                          hn.data_ptr(), cn.data_ptr(), T, B, I, H, ctypes.byref(bufs), prec)
    assert st == 0
    return out.view(T, B, H).cpu(), hn.view(1, B, H).cpu(), cn.view(1, B, H).cpu()


@pytest.mark.parametrize("T,B,I,H", V1_PRESETS)
def test_v1_c_abi_matches_cpu_lstm(T, B, I, H):
    lib = _lib.load()
    torch.manual_seed(T * 1000 + H)
    lstm = torch.nn.LSTM(I, H).eval()
    ACC16 = 1
    bufs = _lib.LstmBuffers()
    assert lib.lstm_create_buffers(ACC16, T, B, I, H, 64, ctypes.byref(bufs)) == 0
    w_ih, w_hh = lstm.weight_ih_l0.detach().cuda().contiguous(), lstm.weight_hh_l0.detach().cuda().contiguous()
    # forward before packing is misuse (src/lstm.cu:1918)
    z = torch.zeros(T * B * max(I, H), device="cuda")
    assert lib.lstm_forward(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
                            z.data_ptr(), z.data_ptr(), T, B, I, H, ctypes.byref(bufs), ACC16) != 0
    assert lib.lstm_pack_weights(ACC16, w_ih.data_ptr(), w_hh.data_ptr(), I, H, ctypes.byref(bufs)) == 0
    assert lib.lstm_pack_weights(0, w_ih.data_ptr(), w_hh.data_ptr(), I, H, ctypes.byref(bufs)) != 0  # precision mismatch
    assert lib.lstm_set_execution_mode(ctypes.byref(bufs), 1) == 0
    # same buffers at T, T/2 and T+1: capacity growth (python/test_lstm.py:186-271)
    for t in (T, max(1, T // 2), T + 1):
        with torch.no_grad():
            x, h0, c0 = torch.randn(t, B, I), torch.randn(1, B, H), torch.randn(1, B, H)
            y_ref, (hn_ref, cn_ref) = lstm(x, (h0, c0))
        y, hn, cn = _v1_forward(lib, bufs, lstm, x, h0, c0, t, B, I, H, ACC16)
        np.testing.assert_allclose(y.numpy(), y_ref.numpy(), atol=1e-3, rtol=5e-2)  # python/test_lstm.py:370-381
        np.testing.assert_allclose(hn.numpy(), hn_ref.numpy(), atol=1e-3, rtol=5e-2)
        np.testing.assert_allclose(cn.numpy(), cn_ref.numpy(), atol=1e-3, rtol=5e-2)
    # wrong batch is rejected
    assert lib.lstm_forward(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
                            z.data_ptr(), z.data_ptr(), T, B + 1, I, H, ctypes.byref(bufs), ACC16) != 0
    assert lib.lstm_destroy_buffers(ctypes.byref(bufs)) == 0
    assert bufs.impl is None


@pytest.mark.parametrize("T,B,I,H,chunk", [(48, 32, 256, 256, 0), (48, 32, 256, 256, 16), (12, 4, 24, 16, 5)])
def test_v1_graph_mode_replays_and_matches_immediate(T, B, I, H, chunk):
    """lstm_set_execution_mode (src/lstm.cu:869-884): GRAPH captures the call and replays it while the sequence
    length and the tensors stay the same, re-records when T changes (:2085-2087); IMMEDIATE launches directly.
    Outputs are bit-identical between the modes and across replays; input_proj_chunk_size splits the sequence
    into ranges without changing a bit either."""
    lib = _lib.load()
    torch.manual_seed(17)
    lstm = torch.nn.LSTM(I, H).eval()
    ACC32, IMMEDIATE, GRAPH = 0, 0, 1
    dev = "cuda"
    w_ih, w_hh = lstm.weight_ih_l0.detach().to(dev).contiguous(), lstm.weight_hh_l0.detach().to(dev).contiguous()
    bi, bh = lstm.bias_ih_l0.detach().to(dev), lstm.bias_hh_l0.detach().to(dev)
    x, h0, c0 = torch.randn(T + 1, B, I, device=dev), torch.randn(B, H, device=dev), torch.randn(B, H, device=dev)
    results = {}
    for mode, ck in ((IMMEDIATE, 0), (GRAPH, chunk)):
        bufs = _lib.LstmBuffers()
        assert lib.lstm_create_buffers(ACC32, T, B, I, H, ck, ctypes.byref(bufs)) == 0
        assert lib.lstm_pack_weights(ACC32, w_ih.data_ptr(), w_hh.data_ptr(), I, H, ctypes.byref(bufs)) == 0
        assert lib.lstm_set_execution_mode(ctypes.byref(bufs), mode) == 0
        out, hn, cn = torch.empty(T + 1, B, H, device=dev), torch.empty(B, H, device=dev), torch.empty(B, H, device=dev)
        runs = []
        for t in (T, T, T, T + 1, T + 1, T):  # replay twice, re-record for T+1, replay, re-record for T
            out.zero_()
            assert lib.lstm_forward(x.data_ptr(), bi.data_ptr(), bh.data_ptr(), h0.data_ptr(), c0.data_ptr(), out.data_ptr(),
                                    hn.data_ptr(), cn.data_ptr(), t, B, I, H, ctypes.byref(bufs), ACC32) == 0
            runs.append((t, out[:t].clone(), hn.clone(), cn.clone()))
        replays = lib.lstm_graph_replays(ctypes.byref(bufs))
        assert replays == (3 if mode == GRAPH else 0)
        assert lib.lstm_destroy_buffers(ctypes.byref(bufs)) == 0
        results[mode] = runs
    for (t, y_i, hn_i, cn_i), (_, y_g, hn_g, cn_g) in zip(results[IMMEDIATE], results[GRAPH]):
        assert torch.equal(y_i, y_g) and torch.equal(hn_i, hn_g) and torch.equal(cn_i, cn_g)
    with torch.no_grad():
        y_ref, _ = lstm(x[:T].cpu(), (h0.cpu().unsqueeze(0), c0.cpu().unsqueeze(0)))
    np.testing.assert_allclose(results[GRAPH][0][1].cpu().numpy(), y_ref.numpy(), atol=1e-3, rtol=5e-2)


def _pinned_half(shape):
    t = torch.empty(shape, dtype=torch.float16, pin_memory=True)
    t.copy_(torch.randn(shape).half())
    return t


def test_streaming_module_matches_torch_lstm():
    """Same construction as the reference's pytest: identical seed before both constructors so the
    parameters coincide; loss = mean(y^2)+mean(hy^2)+mean(cy^2); dx, dh0, dc0 are checked too."""
    from flashlstm_poc_b200.streaming_lstm import StreamingLSTM

    torch.manual_seed(1234)
    T, B, I, H = 4, 2, 3, 5
    module = StreamingLSTM(I, H)
    torch.manual_seed(1234)
    ref = torch.nn.LSTM(I, H, device="cuda")
    assert torch.equal(module.weight_ih, ref.weight_ih_l0) and torch.equal(module.bias_hh, ref.bias_hh_l0)
    x_host = _pinned_half((T, B, I)).requires_grad_(True)
    x_ref = x_host.detach().to("cuda", torch.float32).requires_grad_(True)
    h0 = torch.randn(B, H, device="cuda", dtype=torch.float16, requires_grad=True)
    c0 = torch.randn(B, H, device="cuda", dtype=torch.float16, requires_grad=True)
    h0r = h0.detach().float().unsqueeze(0).requires_grad_(True)
    c0r = c0.detach().float().unsqueeze(0).requires_grad_(True)

    y_host, cache, (hy, cy) = module(x_host, h0, c0)
    assert y_host.is_pinned() and y_host.dtype == torch.float16 and cache.h.shape == (T, B, H)
    y = y_host.to("cuda", torch.float32)
    y_ref, (hy_ref, cy_ref) = ref(x_ref, (h0r, c0r))
    torch.testing.assert_close(y, y_ref, rtol=1e-3, atol=2e-3)
    torch.testing.assert_close(hy.float(), hy_ref[0], rtol=1e-3, atol=2e-3)
    torch.testing.assert_close(cy.float(), cy_ref[0], rtol=1e-3, atol=2e-3)
    # checkpoint semantics: entry k = state entering step k (R = 1); entry 0 = h0/c0
    torch.testing.assert_close(cache.h[0].cuda(), h0.detach().float(), rtol=0, atol=1e-3)
    torch.testing.assert_close(cache.c[0].cuda(), c0.detach().float(), rtol=0, atol=1e-3)
    torch.testing.assert_close(cache.h[1].cuda(), y_ref[0].detach(), rtol=1e-3, atol=2e-3)

    (y.pow(2).mean() + hy.float().pow(2).mean() + cy.float().pow(2).mean()).backward()
    (y_ref.pow(2).mean() + hy_ref.pow(2).mean() + cy_ref.pow(2).mean()).backward()
    for got, want in ((module.weight_ih.grad, ref.weight_ih_l0.grad), (module.weight_hh.grad, ref.weight_hh_l0.grad),
                      (module.bias_ih.grad, ref.bias_ih_l0.grad), (module.bias_hh.grad, ref.bias_hh_l0.grad)):
        torch.testing.assert_close(got, want, rtol=1e-3, atol=5e-3)
    torch.testing.assert_close(x_host.grad.float().cuda(), x_ref.grad, rtol=1e-2, atol=5e-3)
    torch.testing.assert_close(h0.grad.float(), h0r.grad[0], rtol=1e-2, atol=5e-3)
    torch.testing.assert_close(c0.grad.float(), c0r.grad[0], rtol=1e-2, atol=5e-3)


def test_streaming_module_validation_errors():
    from flashlstm_poc_b200.streaming_lstm import StreamingLSTM, streaming_lstm

    m = StreamingLSTM(4, 4)
    with pytest.raises(ValueError, match="pinned"):
        m(torch.zeros(2, 2, 4, dtype=torch.float16))  # pageable host memory
    with pytest.raises(ValueError, match="float16"):
        m(torch.zeros(2, 2, 4).pin_memory())
    x = _pinned_half((2, 2, 4))
    with pytest.raises(ValueError, match="recompute_interval"):
        m(x, recompute_interval=0)
    with pytest.raises(ValueError, match="gate cache dtype"):
        m(x, gate_cache_dtypes=(torch.float64, torch.float32))
    with pytest.raises(ValueError, match="CUDA"):
        m(x, torch.zeros(2, 4, dtype=torch.float16), None)
    with pytest.raises(ValueError, match="weight_ih must have shape"):
        streaming_lstm(x, None, None, m.weight_hh[:, :3].contiguous(), m.weight_hh, m.bias_ih, m.bias_hh)


V2_SHAPES = [(4, 2, 3, 5), (16, 8, 64, 32), (32, 4, 128, 16), (64, 32, 256, 256)]


@pytest.mark.parametrize("T,B,I,H", V2_SHAPES)
@pytest.mark.parametrize("R", [1, 4])
def test_v2_c_abi_forward_backward(T, B, I, H, R):
    """ctypes against the C ABI with the validate scripts' shapes, R=4, fp16 h-checkpoints and
    fp32 c-checkpoints, VJP loss = sum(y dY) + sum(h_n dHN) + sum(c_n dCN) with seed-42 cotangents.
    The reference accepts 5e-2 (forward) and 1e-1 (backward); the bar here is relative L2 <= 1e-2."""
    lib = _lib.load()
    torch.manual_seed(7)
    lstm = torch.nn.LSTM(I, H)
    x = _pinned_half((T, B, I))
    h0, c0 = torch.randn(B, H).half(), torch.randn(B, H).half()
    g = torch.Generator().manual_seed(42)
    dy = torch.randn(T, B, H, generator=g).half().pin_memory()
    dhn, dcn = torch.randn(B, H, generator=g).half(), torch.randn(B, H, generator=g).half()

    # ground truth on the fp16-rounded inputs
    xr = x.float().requires_grad_(True)
    h0r, c0r = h0.float().unsqueeze(0).requires_grad_(True), c0.float().unsqueeze(0).requires_grad_(True)
    y_ref, (hn_ref, cn_ref) = lstm(xr, (h0r, c0r))
    ((y_ref * dy.float()).sum() + (hn_ref[0] * dhn.float()).sum() + (cn_ref[0] * dcn.float()).sum()).backward()

    dev = "cuda"
    P = [p.detach().to(dev).contiguous() for p in (lstm.weight_ih_l0, lstm.weight_hh_l0, lstm.bias_ih_l0, lstm.bias_hh_l0)]
    h0d, c0d = h0.to(dev), c0.to(dev)
    nchk = (T + R - 1) // R
    y = torch.empty(T, B, H, dtype=torch.float16).pin_memory()
    ch = torch.empty(nchk, B, H, dtype=torch.float16).pin_memory()
    cc = torch.empty(nchk, B, H, dtype=torch.float32).pin_memory()
    hy, cy = torch.empty(B, H, dtype=torch.float16, device=dev), torch.empty(B, H, dtype=torch.float16, device=dev)
    s1, s2, s3 = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    opt = _lib.StreamingLstmOptions(1, 0)
    cache = _lib.GateCacheHost(ch.data_ptr(), cc.data_ptr())
    torch.cuda.synchronize()
    lib.flstm_StreamingLstmForward(T, B, I, H, R, x.data_ptr(), h0d.data_ptr(), c0d.data_ptr(), P[0].data_ptr(),
                                   P[1].data_ptr(), P[2].data_ptr(), P[3].data_ptr(), y.data_ptr(), cache,
                                   ctypes.byref(opt), hy.data_ptr(), cy.data_ptr(), s1.cuda_stream, s2.cuda_stream,
                                   s3.cuda_stream)
    assert lib.flstm_last_status() == 0, lib.flstm_last_error()
    assert orc.rel_l2_err(y.float().numpy(), y_ref.detach().numpy()) < 1e-2
    assert orc.rel_l2_err(hy.float().cpu().numpy(), hn_ref[0].detach().numpy()) < 1e-2
    assert orc.rel_l2_err(cy.float().cpu().numpy(), cn_ref[0].detach().numpy()) < 1e-2
    # checkpoints: entry k = state entering step k*R
    assert torch.equal(ch[0], h0)
    for k in range(1, nchk):
        assert orc.rel_l2_err(ch[k].float().numpy(), y_ref[k * R - 1].detach().numpy()) < 1e-2

    dx = torch.empty(T, B, I, dtype=torch.float16).pin_memory()
    G = [torch.empty_like(p) for p in P]
    dh0, dc0 = torch.empty(B, H, device=dev), torch.empty(B, H, device=dev)
    dhnd, dcnd = dhn.to(dev), dcn.to(dev)
    # `options` is the LAST argument of the C backward (flashlstm_v2/include/lstm.hpp:210)
    lib.flstm_StreamingLstmBackward(T, B, I, H, R, x.data_ptr(), y.data_ptr(), cache, dy.data_ptr(), dhnd.data_ptr(),
                                    dcnd.data_ptr(), h0d.data_ptr(), c0d.data_ptr(), P[0].data_ptr(), P[1].data_ptr(),
                                    P[2].data_ptr(), P[3].data_ptr(), dx.data_ptr(), G[0].data_ptr(), G[1].data_ptr(),
                                    G[2].data_ptr(), G[3].data_ptr(), dh0.data_ptr(), dc0.data_ptr(), s1.cuda_stream,
                                    s2.cuda_stream, s3.cuda_stream, ctypes.byref(opt))
    assert lib.flstm_last_status() == 0, lib.flstm_last_error()
    checks = [(dx.float(), xr.grad), (dh0.cpu(), h0r.grad[0]), (dc0.cpu(), c0r.grad[0]),
              (G[0].cpu(), lstm.weight_ih_l0.grad), (G[1].cpu(), lstm.weight_hh_l0.grad),
              (G[2].cpu(), lstm.bias_ih_l0.grad), (G[3].cpu(), lstm.bias_hh_l0.grad)]
    for got, want in checks:
        assert orc.rel_l2_err(got.numpy(), want.numpy()) < 1e-2
    assert torch.equal(G[2], G[3])  # db_ih == db_hh

    # a stateless backward (another forward ran in between) consumes the caller's checkpoints and agrees
    y2 = torch.empty_like(y).pin_memory()
    lib.flstm_StreamingLstmForward(T, B, I, H, R, x.data_ptr(), h0d.data_ptr(), c0d.data_ptr(), P[0].data_ptr(),
                                   P[1].data_ptr(), P[2].data_ptr(), P[3].data_ptr(), y2.data_ptr(), cache,
                                   ctypes.byref(opt), hy.data_ptr(), cy.data_ptr(), s1.cuda_stream, s2.cuda_stream,
                                   s3.cuda_stream)
    G2 = [torch.empty_like(p) for p in P]
    lib.flstm_StreamingLstmBackward(T, B, I, H, R, x.data_ptr(), y.data_ptr(), cache, dy.data_ptr(), dhnd.data_ptr(),
                                    dcnd.data_ptr(), h0d.data_ptr(), c0d.data_ptr(), P[0].data_ptr(), P[1].data_ptr(),
                                    P[2].data_ptr(), P[3].data_ptr(), dx.data_ptr(), G2[0].data_ptr(), G2[1].data_ptr(),
                                    G2[2].data_ptr(), G2[3].data_ptr(), dh0.data_ptr(), dc0.data_ptr(), s1.cuda_stream,
                                    s2.cuda_stream, s3.cuda_stream, ctypes.byref(opt))
    assert lib.flstm_last_status() == 0
    # this one could not use the forward's gate cache: it restored the states from the caller's checkpoints
    # (h fp16 = exact, c fp32 = exact) and recomputed; only the fp32 summation order of dW may differ
    assert orc.rel_l2_err(G2[1].cpu().numpy(), G[1].cpu().numpy()) < 1e-5
    assert orc.rel_l2_err(G2[0].cpu().numpy(), G[0].cpu().numpy()) < 1e-5


def test_v2_rejects_misuse_without_aborting():
    lib = _lib.load()
    s = torch.cuda.Stream()
    z = torch.zeros(64, device="cuda", dtype=torch.float16)
    opt = _lib.StreamingLstmOptions(0, 0)
    cache = _lib.GateCacheHost(z.data_ptr(), z.data_ptr())
    p = z.data_ptr()
    # the three streams must be distinct (flashlstm_v2/src/lstm_forward.cu:500-502)
    lib.flstm_StreamingLstmForward(2, 2, 4, 4, 1, p, p, p, p, p, p, p, p, cache, ctypes.byref(opt), p, p,
                                   s.cuda_stream, s.cuda_stream, s.cuda_stream)
    assert lib.flstm_last_status() == 1 and b"distinct" in lib.flstm_last_error()
    # zero-sized problem: silent no-op (:493-495)
    lib.flstm_StreamingLstmForward(0, 2, 4, 4, 1, p, p, p, p, p, p, p, p, cache, ctypes.byref(opt), p, p, 0, 0, 0)
    assert lib.flstm_last_status() == 0


@pytest.mark.parametrize("recompute_interval", [0, 4])
def test_lstm_module_stacked_bf16_autograd(recompute_interval):
    """nn.LSTM-compatible module: 2 layers, BF16, gradients through autograd vs fp32 torch.nn.LSTM; also with
    activation checkpoints every 4 of the 6 steps."""
    from flashlstm_poc_b200.lstm import LSTM

    torch.manual_seed(3)
    T, B, I, H, L = 6, 8, 64, 64, 2
    m = LSTM(I, H, L, dtype=torch.bfloat16, recompute_interval=recompute_interval)
    ref = torch.nn.LSTM(I, H, L)
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.copy_(p.bfloat16().float()) if "weight" in n else None
            getattr(ref, n).copy_(p.cpu())
    x = torch.randn(T, B, I).bfloat16()
    xg = x.cuda().requires_grad_(True)
    xr = x.float().requires_grad_(True)
    y, (hn, cn) = m(xg)
    yr, (hnr, cnr) = ref(xr)
    dy = torch.randn(T, B, H).bfloat16()
    (y.float() * dy.cuda().float()).sum().backward()
    (yr * dy.float()).sum().backward()
    assert orc.rel_l2_err(y.float().cpu().detach().numpy(), yr.detach().numpy()) < 1e-2
    assert orc.rel_l2_err(xg.grad.float().cpu().numpy(), xr.grad.numpy()) < 1e-2
    for n, p in m.named_parameters():
        assert orc.rel_l2_err(p.grad.cpu().numpy(), getattr(ref, n).grad.numpy()) < 1e-2, n
