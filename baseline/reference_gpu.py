"""ctypes harness that drives EITHER library through the reference's two C ABIs with identical calls:
the rebuilt reference (baseline/_ref/, see build_reference.py) or this repository's drop-in library.
Comparison code only; nothing in the product imports it.

v1 (include/flashlstm/lstm_api.h:23-56): forward only, fp32 device tensors, FP16 tensor-core arithmetic.
v2 (flashlstm_v2/include/lstm.hpp:132-213): forward + backward, pinned-host fp16 x / y / dY / dX, h/c checkpoints."""
from __future__ import annotations

import ctypes
import os
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_V1 = os.path.join(HERE, "_ref", "libflashlstm_v1.so")
REF_V2 = os.path.join(HERE, "_ref", "libflashlstm_v2.so")
OURS = os.path.join(os.path.dirname(HERE), "flashlstm_poc_b200", "libflashlstm_b200.so")

FP16_ACC32, FP16_ACC16 = 0, 1
MODE_IMMEDIATE, MODE_GRAPH = 0, 1


class LstmBuffers(ctypes.Structure):
    _fields_ = [("impl", ctypes.c_void_p)]


class GateCacheHost(ctypes.Structure):
    _fields_ = [("h_ptr", ctypes.c_void_p), ("c_ptr", ctypes.c_void_p)]


class StreamingLstmOptions(ctypes.Structure):
    _fields_ = [("h_dtype", ctypes.c_int), ("c_dtype", ctypes.c_int)]


def load(path: str) -> ctypes.CDLL:
    lib = ctypes.CDLL(path)
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    if hasattr(lib, "lstm_forward"):
        lib.lstm_create_buffers.argtypes = [ci, sz, sz, sz, sz, ci, ctypes.POINTER(LstmBuffers)]
        lib.lstm_destroy_buffers.argtypes = [ctypes.POINTER(LstmBuffers)]
        lib.lstm_set_execution_mode.argtypes = [ctypes.POINTER(LstmBuffers), ci]
        lib.lstm_pack_weights.argtypes = [ci, vp, vp, sz, sz, ctypes.POINTER(LstmBuffers)]
        lib.lstm_forward.argtypes = [vp] * 8 + [sz] * 4 + [ctypes.POINTER(LstmBuffers), ci]
    if hasattr(lib, "flstm_StreamingLstmForward"):
        lib.flstm_StreamingLstmForward.argtypes = [sz] * 5 + [vp] * 8 + [GateCacheHost, ctypes.POINTER(StreamingLstmOptions)] + [vp] * 5
        lib.flstm_StreamingLstmForward.restype = None
        lib.flstm_StreamingLstmBackward.argtypes = [sz] * 5 + [vp, vp, GateCacheHost] + [vp] * 19 + [ctypes.POINTER(StreamingLstmOptions)]
        lib.flstm_StreamingLstmBackward.restype = None
    return lib


class V1Runner:
    """lstm_create_buffers + lstm_pack_weights once, then lstm_forward per call (synchronous)."""

    def __init__(self, lib, T, B, I, H, params, precision=FP16_ACC16, chunk=0, mode=None):
        self.lib, self.dims, self.precision = lib, (T, B, I, H), precision
        self.buf = LstmBuffers()
        rc = lib.lstm_create_buffers(precision, T, B, I, H, chunk, ctypes.byref(self.buf))
        if rc:
            raise RuntimeError(f"lstm_create_buffers -> {rc}")
        if mode is not None:
            rc = lib.lstm_set_execution_mode(ctypes.byref(self.buf), mode)
            if rc:
                raise RuntimeError(f"lstm_set_execution_mode -> {rc}")
        self.w_ih, self.w_hh, self.b_ih, self.b_hh = [p.detach().float().cuda().contiguous() for p in params]
        rc = lib.lstm_pack_weights(precision, self.w_ih.data_ptr(), self.w_hh.data_ptr(), I, H, ctypes.byref(self.buf))
        if rc:
            raise RuntimeError(f"lstm_pack_weights -> {rc}")
        self.y = torch.empty(T, B, H, device="cuda")
        self.hn, self.cn = torch.empty(B, H, device="cuda"), torch.empty(B, H, device="cuda")

    def forward(self, x, h0, c0, T=None):
        T0, B, I, H = self.dims
        T = T or T0
        rc = self.lib.lstm_forward(x.data_ptr(), self.b_ih.data_ptr(), self.b_hh.data_ptr(), h0.data_ptr(), c0.data_ptr(),
                                   self.y.data_ptr(), self.hn.data_ptr(), self.cn.data_ptr(), T, B, I, H,
                                   ctypes.byref(self.buf), self.precision)
        if rc:
            raise RuntimeError(f"lstm_forward -> {rc}")
        return self.y[:T], self.hn, self.cn

    def close(self):
        self.lib.lstm_destroy_buffers(ctypes.byref(self.buf))


class V2Runner:
    """flstm_StreamingLstmForward / Backward with pinned host tensors and three streams, as the reference's
    validate scripts call them (flashlstm_v2/scripts/validate_lstm_fwd.py:194-215, validate_lstm_bwd.py:333-363)."""

    def __init__(self, lib, T, B, I, H, R, params, x, h0, c0, dy, h_dtype=1, c_dtype=0):
        self.lib, self.dims, self.R = lib, (T, B, I, H), R
        dev = "cuda"
        self.P = [p.detach().float().to(dev).contiguous() for p in params]
        self.x = x.half().contiguous().pin_memory()
        self.dy = dy.half().contiguous().pin_memory()
        self.h0, self.c0 = h0.half().to(dev).contiguous(), c0.half().to(dev).contiguous()
        n = (T + R - 1) // R
        self.y = torch.empty(T, B, H, dtype=torch.float16).pin_memory()
        self.ch = torch.empty(n, B, H, dtype=torch.float16 if h_dtype else torch.float32).pin_memory()
        self.cc = torch.empty(n, B, H, dtype=torch.float16 if c_dtype else torch.float32).pin_memory()
        self.hy, self.cy = torch.empty_like(self.h0), torch.empty_like(self.c0)
        self.dx = torch.empty(T, B, I, dtype=torch.float16).pin_memory()
        self.G = [torch.empty_like(p) for p in self.P]
        self.dh0, self.dc0 = torch.empty(B, H, device=dev), torch.empty(B, H, device=dev)
        self.streams = [torch.cuda.Stream() for _ in range(3)]
        self.opt = StreamingLstmOptions(h_dtype, c_dtype)
        self.cache = GateCacheHost(self.ch.data_ptr(), self.cc.data_ptr())
        torch.cuda.synchronize()

    def forward(self):
        T, B, I, H = self.dims
        P, s = self.P, self.streams
        self.lib.flstm_StreamingLstmForward(T, B, I, H, self.R, self.x.data_ptr(), self.h0.data_ptr(), self.c0.data_ptr(),
                                            P[0].data_ptr(), P[1].data_ptr(), P[2].data_ptr(), P[3].data_ptr(),
                                            self.y.data_ptr(), self.cache, ctypes.byref(self.opt), self.hy.data_ptr(),
                                            self.cy.data_ptr(), s[0].cuda_stream, s[1].cuda_stream, s[2].cuda_stream)

    def backward(self, dhn=None, dcn=None):
        T, B, I, H = self.dims
        P, G, s = self.P, self.G, self.streams
        self.lib.flstm_StreamingLstmBackward(T, B, I, H, self.R, self.x.data_ptr(), self.y.data_ptr(), self.cache,
                                             self.dy.data_ptr(), None if dhn is None else dhn.data_ptr(),
                                             None if dcn is None else dcn.data_ptr(), self.h0.data_ptr(), self.c0.data_ptr(),
                                             P[0].data_ptr(), P[1].data_ptr(), P[2].data_ptr(), P[3].data_ptr(),
                                             self.dx.data_ptr(), G[0].data_ptr(), G[1].data_ptr(), G[2].data_ptr(),
                                             G[3].data_ptr(), self.dh0.data_ptr(), self.dc0.data_ptr(), s[0].cuda_stream,
                                             s[1].cuda_stream, s[2].cuda_stream, ctypes.byref(self.opt))


def time_calls(fn, warmup: int, iters: int) -> float:
    """Median seconds per call; the calls are synchronous, so the host clock between synchronised points is
    what the reference's own benchmark measures (python/benchmark_lstm.py:185-194)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(iters):
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        samples.append(time.perf_counter() - t0)
    samples.sort()
    return samples[len(samples) // 2]
