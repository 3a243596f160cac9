"""The reference's Python operator for this path, on the B200 engine.

Public names, argument meaning, return values and error behaviour follow
flashlstm_v2/python/flashlstm/streaming_lstm.py: `GateCache` (:14-16), the autograd function
(:61-344), `streaming_lstm` (:347-376) and `StreamingLSTM` (:379-430).  The contract:

* x is a pinned CPU fp16 tensor (T,B,I); h0/c0 are CUDA fp16 (B,H) or None (zeros);
  parameters are CUDA fp32; y comes back as pinned CPU fp16; the two checkpoint tensors
  ("gate cache": state entering step k*R) are pinned, fp32 or fp16, non-differentiable;
  hy/cy are CUDA fp16.
* backward returns dx as pinned CPU fp16, dh0/dc0 cast to the state dtype, fp32 parameter
  gradients, with db_ih == db_hh.
* wrong devices / dtypes / shapes raise ValueError.

The native calls go through the `_flashlstm` extension exactly as in the reference (22 and 30
integer arguments).  A CUDA (device) tensor is also accepted for x and is used in place.
"""

from __future__ import annotations

import math
from typing import NamedTuple, Optional, Tuple

import torch
from torch import nn

from ._flashlstm import streaming_lstm_backward as _native_backward
from ._flashlstm import streaming_lstm_forward as _native_forward

_CACHE_DTYPE_CODE = {torch.float32: 0, torch.float16: 1}


class GateCache(NamedTuple):
    h: torch.Tensor
    c: torch.Tensor


def _cache_code(dtype: torch.dtype) -> int:
    try:
        return _CACHE_DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"gate cache dtype must be float16 or float32, got {dtype}") from None


def _require_host_tensor(t: torch.Tensor, name: str, dtype: torch.dtype) -> None:
    """x / y / dY / checkpoints live in pinned host memory (a CUDA tensor is tolerated)."""
    if t.dtype != dtype:
        raise ValueError(f"{name} must use dtype {dtype}, got {t.dtype}.")
    if t.device.type == "cuda":
        return
    if t.device.type != "cpu":
        raise ValueError(f"{name} must reside on the CPU (pinned host memory).")
    if not t.is_pinned():
        raise ValueError(f"{name} must be allocated in pinned memory (tensor.pin_memory()).")


def _state_or_zeros(t: Optional[torch.Tensor], shape: Tuple[int, int], name: str) -> torch.Tensor:
    if t is None:
        return torch.zeros(shape, device="cuda", dtype=torch.float16)
    if t.device.type != "cuda":
        raise ValueError(f"{name} must reside on CUDA, got device {t.device}.")
    if t.dtype != torch.float16:
        raise ValueError(f"{name} must use dtype torch.float16, got {t.dtype}.")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    return t.contiguous()


def _three_streams():
    return torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()


def _host_like(t: torch.Tensor, shape, dtype) -> torch.Tensor:
    """Output buffer where the caller's x lives: pinned host memory, or the same CUDA device."""
    if t.device.type == "cuda":
        return torch.empty(shape, dtype=dtype, device=t.device)
    return torch.empty(shape, dtype=dtype, pin_memory=True)


class _StreamingLSTMFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_host, h0, c0, weight_ih, weight_hh, bias_ih, bias_hh, recompute_interval, gate_cache_dtypes):
        _require_host_tensor(x_host, "x_host", torch.float16)
        x_host = x_host.contiguous()
        if recompute_interval <= 0:
            raise ValueError(f"recompute_interval must be >= 1, got {recompute_interval}")
        for name, p in (("weight_ih", weight_ih), ("weight_hh", weight_hh), ("bias_ih", bias_ih), ("bias_hh", bias_hh)):
            if p.device.type != "cuda":
                raise ValueError(f"{name} must reside on CUDA.")
            if p.dtype != torch.float32:
                raise ValueError(f"{name} must use dtype torch.float32.")
        T, B, I = x_host.shape
        H = weight_hh.size(1)
        G = 4 * H
        if tuple(weight_ih.shape) != (G, I):
            raise ValueError(f"weight_ih must have shape {(G, I)}, got {tuple(weight_ih.shape)}")
        if tuple(weight_hh.shape) != (G, H):
            raise ValueError(f"weight_hh must have shape {(G, H)}, got {tuple(weight_hh.shape)}")
        if bias_ih.numel() != G or bias_hh.numel() != G:
            raise ValueError("Bias tensors must have length 4 * hidden_size.")
        h0 = _state_or_zeros(h0, (B, H), "h0")
        c0 = _state_or_zeros(c0, (B, H), "c0")
        h_dtype, c_dtype = gate_cache_dtypes
        h_code, c_code = _cache_code(h_dtype), _cache_code(c_dtype)
        n_chk = (T + recompute_interval - 1) // recompute_interval

        y_host = _host_like(x_host, (T, B, H), torch.float16)
        cache_h = _host_like(x_host, (n_chk, B, H), h_dtype)
        cache_c = _host_like(x_host, (n_chk, B, H), c_dtype)
        hy = torch.empty((B, H), device="cuda", dtype=torch.float16)
        cy = torch.empty_like(hy)
        w_ih, w_hh = weight_ih.detach().contiguous(), weight_hh.detach().contiguous()
        b_ih, b_hh = bias_ih.detach().contiguous(), bias_hh.detach().contiguous()

        compute, h2d, d2h = _three_streams()
        compute.wait_stream(torch.cuda.current_stream())
        _native_forward(
            T, B, I, H, recompute_interval, x_host.data_ptr(), h0.data_ptr(), c0.data_ptr(), w_ih.data_ptr(),
            w_hh.data_ptr(), b_ih.data_ptr(), b_hh.data_ptr(), y_host.data_ptr(), cache_h.data_ptr(),
            cache_c.data_ptr(), h_code, c_code, hy.data_ptr(), cy.data_ptr(), compute.cuda_stream, h2d.cuda_stream,
            d2h.cuda_stream,
        )
        torch.cuda.current_stream().wait_stream(compute)

        ctx.save_for_backward(x_host, h0, c0, weight_ih, weight_hh, bias_ih, bias_hh, y_host, cache_h, cache_c)
        ctx.meta = (T, B, I, H, recompute_interval, h_code, c_code)
        ctx.mark_non_differentiable(cache_h, cache_c)
        return y_host, cache_h, cache_c, hy, cy

    @staticmethod
    def backward(ctx, grad_y, _grad_cache_h, _grad_cache_c, grad_hy, grad_cy):
        x_host, h0, c0, weight_ih, weight_hh, bias_ih, bias_hh, y_host, cache_h, cache_c = ctx.saved_tensors
        T, B, I, H, R, h_code, c_code = ctx.meta
        for name, t in (("gate_cache_h", cache_h), ("gate_cache_c", cache_c)):
            if t.dtype not in _CACHE_DTYPE_CODE:
                raise ValueError(f"Unsupported dtype for {name}: {t.dtype}")
            _require_host_tensor(t, name, t.dtype)

        if grad_y is None:
            grad_y = torch.zeros_like(y_host)
        else:
            if grad_y.device != y_host.device:
                raise ValueError("grad_y_host must reside on the CPU." if y_host.device.type == "cpu"
                                 else "grad_y must reside where y does.")
            grad_y = grad_y.to(dtype=torch.float16).contiguous()
            if grad_y.device.type == "cpu" and not grad_y.is_pinned():
                grad_y = grad_y.pin_memory()
        _require_host_tensor(grad_y, "grad_y_host", torch.float16)

        def state_grad(g, name):
            if g is None:
                return None, 0
            if g.device.type != "cuda":
                raise ValueError(f"{name} must reside on CUDA.")
            g = g.to(dtype=torch.float16).contiguous()
            return g, g.data_ptr()

        grad_hy, grad_hy_ptr = state_grad(grad_hy, "grad_hy")
        grad_cy, grad_cy_ptr = state_grad(grad_cy, "grad_cy")

        dx_host = _host_like(x_host, tuple(x_host.shape), torch.float16)
        dw_ih = torch.zeros_like(weight_ih, memory_format=torch.contiguous_format)
        dw_hh = torch.zeros_like(weight_hh, memory_format=torch.contiguous_format)
        db_ih = torch.zeros_like(bias_ih, memory_format=torch.contiguous_format)
        db_hh = torch.zeros_like(bias_hh, memory_format=torch.contiguous_format)
        dh0 = torch.empty((B, H), device="cuda", dtype=torch.float32)
        dc0 = torch.empty_like(dh0)
        w_ih, w_hh = weight_ih.detach().contiguous(), weight_hh.detach().contiguous()
        b_ih, b_hh = bias_ih.detach().contiguous(), bias_hh.detach().contiguous()

        compute, h2d, d2h = _three_streams()
        compute.wait_stream(torch.cuda.current_stream())
        _native_backward(
            T, B, I, H, R, x_host.data_ptr(), y_host.data_ptr(), cache_h.data_ptr(), cache_c.data_ptr(), h_code,
            c_code, grad_y.data_ptr(), grad_hy_ptr, grad_cy_ptr, h0.data_ptr(), c0.data_ptr(), w_ih.data_ptr(),
            w_hh.data_ptr(), b_ih.data_ptr(), b_hh.data_ptr(), dx_host.data_ptr(), dw_ih.data_ptr(),
            dw_hh.data_ptr(), db_ih.data_ptr(), db_hh.data_ptr(), dh0.data_ptr(), dc0.data_ptr(),
            compute.cuda_stream, h2d.cuda_stream, d2h.cuda_stream,
        )
        torch.cuda.current_stream().wait_stream(compute)
        return dx_host, dh0.to(h0.dtype), dc0.to(c0.dtype), dw_ih, dw_hh, db_ih, db_hh, None, None


def streaming_lstm(
    x_host: torch.Tensor,
    h0: Optional[torch.Tensor],
    c0: Optional[torch.Tensor],
    weight_ih: torch.Tensor,
    weight_hh: torch.Tensor,
    bias_ih: torch.Tensor,
    bias_hh: torch.Tensor,
    *,
    recompute_interval: int = 1,
    gate_cache_dtypes: Tuple[torch.dtype, torch.dtype] = (torch.float32, torch.float32),
) -> Tuple[torch.Tensor, GateCache, torch.Tensor, torch.Tensor]:
    """Functional form: returns (y_host, GateCache(h, c), hy, cy)."""
    y, ch, cc, hy, cy = _StreamingLSTMFunction.apply(
        x_host, h0, c0, weight_ih, weight_hh, bias_ih, bias_hh, recompute_interval, gate_cache_dtypes
    )
    return y, GateCache(ch, cc), hy, cy


class StreamingLSTM(nn.Module):
    """Single-layer LSTM module with fp32 CUDA parameters drawn from U(-1/sqrt(H), 1/sqrt(H)) in
    the order weight_ih, weight_hh, bias_ih, bias_hh (torch.nn.LSTM's order, which the
    reference's test relies on: flashlstm_v2/python/tests/test_streaming_lstm.py:15-26)."""

    def __init__(self, input_size: int, hidden_size: int) -> None:
        super().__init__()
        self.input_size, self.hidden_size = int(input_size), int(hidden_size)
        G = 4 * self.hidden_size
        mk = lambda *shape: nn.Parameter(torch.empty(*shape, device="cuda", dtype=torch.float32))
        self.weight_ih = mk(G, self.input_size)
        self.weight_hh = mk(G, self.hidden_size)
        self.bias_ih = mk(G)
        self.bias_hh = mk(G)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        bound = 1.0 / math.sqrt(self.hidden_size) if self.hidden_size > 0 else 0.0
        for p in self.parameters():
            nn.init.uniform_(p, -bound, bound)

    def forward(self, x_host, h0=None, c0=None, *, recompute_interval: int = 1,
                gate_cache_dtypes: Tuple[torch.dtype, torch.dtype] = (torch.float32, torch.float32)):
        _require_host_tensor(x_host, "x_host", torch.float16)
        B = x_host.size(1)
        h0 = _state_or_zeros(h0, (B, self.hidden_size), "h0")
        c0 = _state_or_zeros(c0, (B, self.hidden_size), "c0")
        y, cache, hy, cy = streaming_lstm(
            x_host, h0, c0, self.weight_ih, self.weight_hh, self.bias_ih, self.bias_hh,
            recompute_interval=recompute_interval, gate_cache_dtypes=gate_cache_dtypes,
        )
        return y, cache, (hy, cy)
