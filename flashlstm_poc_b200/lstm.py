"""`LSTM`: a torch.nn.LSTM-compatible module (seq-major, unidirectional, stacked layers) whose
forward and backward run on the B200 engine with device-resident tensors.  This is the surface
for what the reference's operator cannot express: stacked layers, BF16 and batch-sharded data
parallelism with the weight-gradient allreduce inside the backward pass."""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import nn

from .engine import DTYPE_OF_TORCH, Engine


class _LSTMFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, module, x, h0, c0, *params):
        eng = module._engine_for(x)
        for l in range(module.num_layers):
            eng.set_weights(l, *params[4 * l:4 * l + 4])
        y, hn, cn = eng.forward(x, h0, c0)
        ctx.module, ctx.engine = module, eng
        ctx.has_h0, ctx.has_c0 = h0 is not None, c0 is not None
        ctx.state_dtype = x.dtype
        return y, hn, cn

    @staticmethod
    def backward(ctx, dy, dhn, dcn):
        eng = ctx.engine
        if dy is None:
            raise RuntimeError("LSTM backward needs a gradient for y")
        dx, dh0, dc0 = eng.backward(dy.contiguous(), dhn, dcn)
        grads = []
        for l in range(ctx.module.num_layers):
            dw_ih, dw_hh, db = eng.grads(l)
            grads += [dw_ih.clone(), dw_hh.clone(), db.clone(), db.clone()]
        return (None, dx, dh0.to(ctx.state_dtype) if ctx.has_h0 else None,
                dc0.to(ctx.state_dtype) if ctx.has_c0 else None, *grads)


class LSTM(nn.Module):
    """Drop-in for torch.nn.LSTM(input_size, hidden_size, num_layers) (bias=True,
    batch_first=False, no dropout, no projection, unidirectional).  Parameters are fp32 and
    named as in torch.nn.LSTM (weight_ih_l{k}, ...); `dtype` selects the engine's arithmetic."""

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, *, dtype: torch.dtype = torch.float16,
                 device="cuda", backend: str = "auto", recompute_interval: int = 0):
        super().__init__()
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.compute_dtype, self.backend = dtype, backend
        # > 0: activation checkpoints every `recompute_interval` steps instead of a full gate cache (the
        # reference's recompute_interval, flashlstm_v2/python/flashlstm/streaming_lstm.py:356)
        self.recompute_interval = int(recompute_interval)
        bound = 1.0 / math.sqrt(hidden_size)
        for l in range(num_layers):
            I = input_size if l == 0 else hidden_size
            for name, shape in ((f"weight_ih_l{l}", (4 * hidden_size, I)), (f"weight_hh_l{l}", (4 * hidden_size, hidden_size)),
                                (f"bias_ih_l{l}", (4 * hidden_size,)), (f"bias_hh_l{l}", (4 * hidden_size,))):
                p = nn.Parameter(torch.empty(shape, device=device, dtype=torch.float32))
                nn.init.uniform_(p, -bound, bound)
                self.register_parameter(name, p)
        self._engines = {}
        self._comm = None

    def _flat_params(self):
        out = []
        for l in range(self.num_layers):
            out += [getattr(self, f"weight_ih_l{l}"), getattr(self, f"weight_hh_l{l}"),
                    getattr(self, f"bias_ih_l{l}"), getattr(self, f"bias_hh_l{l}")]
        return out

    def _engine_for(self, x: torch.Tensor) -> Engine:
        T, B, _ = x.shape
        key = (B, x.device.index)
        eng = self._engines.get(key)
        if eng is None:
            eng = Engine(DTYPE_OF_TORCH[self.compute_dtype], self.num_layers, B, self.input_size, self.hidden_size, T,
                         training=True, backend=self.backend, device=x.device)
            if self.recompute_interval:
                eng.set_recompute_interval(self.recompute_interval)
            if self._comm is not None:
                eng.attach_comm(*self._comm)
            self._engines[key] = eng
        return eng

    def attach_comm(self, unique_id: bytes, rank: int, world_size: int) -> None:
        """Batch-sharded data parallelism: every rank's weight gradients are summed inside backward."""
        self._comm = (unique_id, rank, world_size)
        for eng in self._engines.values():
            eng.attach_comm(unique_id, rank, world_size)

    def forward(self, x: torch.Tensor, hx: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        if x.dtype != self.compute_dtype:
            raise ValueError(f"x must have dtype {self.compute_dtype}, got {x.dtype}")
        h0, c0 = hx if hx is not None else (None, None)
        y, hn, cn = _LSTMFunction.apply(self, x.contiguous(), h0, c0, *self._flat_params())
        return y, (hn, cn)
