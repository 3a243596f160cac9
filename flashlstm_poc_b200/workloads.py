"""Seeded synthetic workloads: the five benchmark configurations and their inputs.

The reference ships no dataset; its benchmarks and tests draw seeded random tensors
(python/benchmark_lstm.py:185-194, flashlstm_v2/src/main.cu:280-285).  The same is done
here, with one fixed generation order per seed so every consumer (tests, benchmark,
CPU baseline) sees identical values:

    torch.manual_seed(seed)
    nn.LSTM(I, H, L) construction  -> weight_ih, weight_hh, bias_ih, bias_hh per layer,
                                      U(-1/sqrt(H), 1/sqrt(H))  (nn.LSTM init order)
    x ~ N(0,1) (T,B,I);  h0, c0 ~ N(0, state_std) (L,B,H) or zeros;  dY ~ N(0,1) (T,B,H)

For 16-bit configurations x, the weights, h0, c0 and dY are rounded once to the 16-bit
type and the ROUNDED values are what both the engine and the fp32 CPU ground truth
consume (biases stay fp32), so a comparison measures arithmetic, not input quantisation
(the reference's own test does the same, flashlstm_v2/python/tests/test_streaming_lstm.py:28-34).
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict, List, Optional

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    dtype: str  # "f32" | "f16" | "bf16"
    layers: int
    input_size: int
    hidden_size: int
    batch: int
    seq_len: int
    seed: int
    state_std: float = 0.0  # 0 -> h0 = c0 = 0
    training: bool = True

    @property
    def tokens(self) -> int:
        return self.batch * self.seq_len

    def flops(self) -> float:
        """Algorithmic FLOPs of one step: 24*T*B*H*sum_l(I_l+H) for training, a third of
        that for inference (pointwise excluded: flashlstm_v2/include/mfu_profiler.hpp:13-15)."""
        z = 0
        for l in range(self.layers):
            z += (self.input_size if l == 0 else self.hidden_size) + self.hidden_size
        full = 24.0 * self.seq_len * self.batch * self.hidden_size * z
        return full if self.training else full / 3.0

    def scaled(self, **kw) -> "Workload":
        return replace(self, **kw)


WORKLOADS: Dict[str, Workload] = {
    "c1_fp32_h256": Workload("c1_fp32_h256", "f32", 1, 256, 256, 32, 128, seed=0),
    "c2_fp16_h1024": Workload("c2_fp16_h1024", "f16", 1, 1024, 1024, 64, 512, seed=1, state_std=0.1),
    "c3_bf16_l2_h2048": Workload("c3_bf16_l2_h2048", "bf16", 2, 2048, 2048, 256, 1024, seed=2),
    "c4_fp16_h4096_b1": Workload("c4_fp16_h4096_b1", "f16", 1, 4096, 4096, 1, 2048, seed=3, training=False),
    "c4_fp16_h4096_b8": Workload("c4_fp16_h4096_b8", "f16", 1, 4096, 4096, 8, 2048, seed=3, training=False),
    "c5_bf16_l4_h1024": Workload("c5_bf16_l4_h1024", "bf16", 4, 1024, 1024, 2048, 256, seed=4),
}

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


@dataclass
class Inputs:
    """fp32 CPU tensors whose values are exactly representable in the workload dtype."""

    w_ih: List[torch.Tensor]
    w_hh: List[torch.Tensor]
    b_ih: List[torch.Tensor]
    b_hh: List[torch.Tensor]
    x: torch.Tensor
    h0: Optional[torch.Tensor]
    c0: Optional[torch.Tensor]
    dy: Optional[torch.Tensor]


def _round_to(t: torch.Tensor, dtype: str) -> torch.Tensor:
    if dtype == "f32":
        return t
    return t.to(TORCH_DTYPE[dtype]).to(torch.float32)


def make_inputs(w: Workload, rows: Optional[slice] = None) -> Inputs:
    """`rows` keeps only that slice of the batch (the draw itself is always the full batch, so every rank of a
    batch-sharded run sees the values a single-GPU run sees for the same sequences)."""
    torch.manual_seed(w.seed)
    proto = torch.nn.LSTM(w.input_size, w.hidden_size, num_layers=w.layers)
    w_ih, w_hh, b_ih, b_hh = [], [], [], []
    for l in range(w.layers):
        w_ih.append(_round_to(getattr(proto, f"weight_ih_l{l}").detach().clone(), w.dtype))
        w_hh.append(_round_to(getattr(proto, f"weight_hh_l{l}").detach().clone(), w.dtype))
        b_ih.append(getattr(proto, f"bias_ih_l{l}").detach().clone())
        b_hh.append(getattr(proto, f"bias_hh_l{l}").detach().clone())
    def keep(t: torch.Tensor) -> torch.Tensor:
        return t if rows is None else t[:, rows].contiguous()

    x = keep(_round_to(torch.randn(w.seq_len, w.batch, w.input_size), w.dtype))
    if w.state_std > 0:
        h0 = keep(_round_to(torch.randn(w.layers, w.batch, w.hidden_size) * w.state_std, w.dtype))
        c0 = keep(_round_to(torch.randn(w.layers, w.batch, w.hidden_size) * w.state_std, w.dtype))
    else:
        h0 = c0 = None
    dy = keep(_round_to(torch.randn(w.seq_len, w.batch, w.hidden_size), w.dtype)) if w.training else None
    return Inputs(w_ih, w_hh, b_ih, b_hh, x, h0, c0, dy)


def shard_batch(t: Optional[torch.Tensor], rank: int, world: int, dim: int = 1) -> Optional[torch.Tensor]:
    """Contiguous slice of the batch dimension owned by `rank` (batch-sharded data parallel)."""
    if t is None:
        return None
    per = t.shape[dim] // world
    return t.narrow(dim, rank * per, per).contiguous()
