"""CPU oracle for the LSTM forward/backward hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker that the CUDA engine is compared with.  It is never
part of the product path: only the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it.

It is a plain-numpy restatement of the algorithm the reference states in its own
CPU code (one GEMM plus one fused pointwise op per time step, a full i/f/g/o + c
cache, a reverse loop with one GEMM per step and one deferred parameter GEMM):

* forward pointwise  -> flashlstm_v2/playground/simple_lstm_bwd.py:28-49
* backward pointwise -> flashlstm_v2/playground/simple_lstm_bwd.py:52-90
* weight concat / bias fuse -> flashlstm_v2/playground/simple_lstm_bwd.py:105-115
* forward loop + cache contents -> flashlstm_v2/playground/simple_lstm_bwd.py:122-176
* backward loop, deferred dW GEMM, db_ih == db_hh -> simple_lstm_bwd.py:187-260
* h/c checkpoint ("gate cache") semantics, i.e. the state ENTERING step k*R
  -> flashlstm_v2/src/lstm_forward.cu:727-783 (+ :370-375)
* stacked layers follow torch.nn.LSTM(num_layers=L): layer l consumes y of layer l-1.

Parity is pinned two ways (tests/test_oracle.py): against golden vectors generated
by importing the reference's playground code (tests/golden/make_golden.py) and
against torch.nn.LSTM forward + autograd.

Semantics: PyTorch nn.LSTM.  Gate row order i, f, g, o in every (4H, .) tensor;
two biases that are summed; seq-major (T, B, .) tensors.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np


def _sigmoid(a: np.ndarray) -> np.ndarray:
    # numerically safe for large |a| in either sign
    out = np.empty_like(a)
    pos = a >= 0
    out[pos] = 1.0 / (1.0 + np.exp(-a[pos]))
    e = np.exp(a[~pos])
    out[~pos] = e / (1.0 + e)
    return out


@dataclass
class LayerParams:
    """One layer's parameters in torch.nn.LSTM layout."""

    w_ih: np.ndarray  # (4H, I_l)
    w_hh: np.ndarray  # (4H, H)
    b_ih: np.ndarray  # (4H,)
    b_hh: np.ndarray  # (4H,)


@dataclass
class LayerCache:
    """Everything the backward loop of one layer consumes (simple_lstm_bwd.py:141-176)."""

    x: np.ndarray  # (T, B, I_l) layer input
    h_s: np.ndarray  # (T+1, B, H); slot 0 = h0, slot t+1 = h_t
    c_s: np.ndarray  # (T+1, B, H); slot 0 = c0
    gates: np.ndarray  # (T, B, 4H) post-activation i,f,g,o


@dataclass
class ForwardResult:
    y: np.ndarray  # (T, B, H) output of the last layer
    h_n: np.ndarray  # (L, B, H)
    c_n: np.ndarray  # (L, B, H)
    caches: List[LayerCache] = field(default_factory=list)


@dataclass
class BackwardResult:
    dx: np.ndarray  # (T, B, I)
    dh0: np.ndarray  # (L, B, H)
    dc0: np.ndarray  # (L, B, H)
    dw_ih: List[np.ndarray]
    dw_hh: List[np.ndarray]
    db_ih: List[np.ndarray]
    db_hh: List[np.ndarray]
    dgates: List[np.ndarray]  # per layer (T, B, 4H) pre-activation gradients


def pointwise_forward(pre: np.ndarray, c_prev: np.ndarray):
    """Fused forward pointwise for one step (simple_lstm_bwd.py:28-49).

    pre: (B, 4H) pre-activations, gate order i,f,g,o.  Returns h, c, act(B,4H)."""
    H = pre.shape[1] // 4
    i = _sigmoid(pre[:, 0:H])
    f = _sigmoid(pre[:, H : 2 * H])
    g = np.tanh(pre[:, 2 * H : 3 * H])
    o = _sigmoid(pre[:, 3 * H : 4 * H])
    c = f * c_prev + i * g
    h = o * np.tanh(c)
    return h, c, np.concatenate([i, f, g, o], axis=1)


def pointwise_backward(dh, dc_next, act, c_t, c_prev):
    """Fused backward pointwise for one step (simple_lstm_bwd.py:52-90).

    Returns dG (B,4H) pre-activation gradients and dc_prev (B,H)."""
    H = c_t.shape[1]
    i = act[:, 0:H]
    f = act[:, H : 2 * H]
    g = act[:, 2 * H : 3 * H]
    o = act[:, 3 * H : 4 * H]
    tanh_c = np.tanh(c_t)
    do = dh * tanh_c
    dc = dc_next + dh * o * (1.0 - tanh_c * tanh_c)
    dai = dc * g * i * (1.0 - i)
    daf = dc * c_prev * f * (1.0 - f)
    dag = dc * i * (1.0 - g * g)
    dao = do * o * (1.0 - o)
    return np.concatenate([dai, daf, dag, dao], axis=1), dc * f


def lstm_forward(
    x: np.ndarray,
    params: Sequence[LayerParams],
    h0: Optional[np.ndarray] = None,
    c0: Optional[np.ndarray] = None,
    dtype=np.float32,
    keep_cache: bool = True,
) -> ForwardResult:
    """Stacked LSTM forward.  x (T,B,I); h0/c0 (L,B,H) or None for zeros."""
    x = np.ascontiguousarray(x, dtype=dtype)
    T, B, _ = x.shape
    L = len(params)
    H = params[0].w_hh.shape[1]
    h_n = np.zeros((L, B, H), dtype=dtype)
    c_n = np.zeros((L, B, H), dtype=dtype)
    caches: List[LayerCache] = []
    layer_in = x
    for l, p in enumerate(params):
        # concat weights so each step is ONE GEMM (simple_lstm_bwd.py:105-115)
        w_cat = np.concatenate([p.w_ih.T, p.w_hh.T], axis=0).astype(dtype)  # (I+H, 4H)
        bias = (p.b_ih.astype(dtype) + p.b_hh.astype(dtype)).astype(dtype)
        h = np.zeros((B, H), dtype) if h0 is None else np.array(h0[l], dtype=dtype)
        c = np.zeros((B, H), dtype) if c0 is None else np.array(c0[l], dtype=dtype)
        h_s = np.empty((T + 1, B, H), dtype)
        c_s = np.empty((T + 1, B, H), dtype)
        gates = np.empty((T, B, 4 * H), dtype)
        h_s[0], c_s[0] = h, c
        for t in range(T):
            z = np.concatenate([layer_in[t], h], axis=1)
            pre = z @ w_cat + bias
            h, c, act = pointwise_forward(pre, c)
            h_s[t + 1], c_s[t + 1], gates[t] = h, c, act
        h_n[l], c_n[l] = h, c
        if keep_cache:
            caches.append(LayerCache(layer_in, h_s, c_s, gates))
        layer_in = h_s[1:]
    return ForwardResult(np.ascontiguousarray(layer_in), h_n, c_n, caches)


def lstm_backward(
    fwd: ForwardResult,
    params: Sequence[LayerParams],
    dy: np.ndarray,
    dh_n: Optional[np.ndarray] = None,
    dc_n: Optional[np.ndarray] = None,
    dtype=np.float32,
) -> BackwardResult:
    """Stacked LSTM backward (BPTT), layers from top to bottom.

    dy (T,B,H) gradient of the last layer's output; dh_n/dc_n (L,B,H) or None."""
    L = len(params)
    T, B, H = fwd.caches[0].h_s.shape[0] - 1, fwd.y.shape[1], fwd.y.shape[2]
    d_out = np.ascontiguousarray(dy, dtype=dtype)
    dh0 = np.zeros((L, B, H), dtype)
    dc0 = np.zeros((L, B, H), dtype)
    dw_ih = [None] * L
    dw_hh = [None] * L
    db = [None] * L
    dgs = [None] * L
    for l in reversed(range(L)):
        p, cache = params[l], fwd.caches[l]
        I = cache.x.shape[2]
        w_hh = p.w_hh.astype(dtype)
        w_ih = p.w_ih.astype(dtype)
        dh_next = np.zeros((B, H), dtype) if dh_n is None else np.array(dh_n[l], dtype=dtype)
        dc_next = np.zeros((B, H), dtype) if dc_n is None else np.array(dc_n[l], dtype=dtype)
        dG = np.empty((T, B, 4 * H), dtype)
        for t in reversed(range(T)):
            dh = d_out[t] + dh_next
            dG[t], dc_next = pointwise_backward(
                dh, dc_next, cache.gates[t], cache.c_s[t + 1], cache.c_s[t]
            )
            dh_next = dG[t] @ w_hh  # (B,4H)@(4H,H)
        dh0[l], dc0[l] = dh_next, dc_next
        flat = dG.reshape(T * B, 4 * H)
        # deferred parameter GEMMs over the whole sequence (simple_lstm_bwd.py:240-252)
        dw_ih[l] = flat.T @ cache.x.reshape(T * B, I)
        dw_hh[l] = flat.T @ cache.h_s[:T].reshape(T * B, H)
        db[l] = flat.sum(axis=0)
        dgs[l] = dG
        d_out = (flat @ w_ih).reshape(T, B, I)  # dX of this layer = dY of the layer below
    return BackwardResult(
        dx=d_out, dh0=dh0, dc0=dc0, dw_ih=dw_ih, dw_hh=dw_hh,
        db_ih=[b.copy() for b in db], db_hh=[b.copy() for b in db], dgates=dgs,
    )


def checkpoints(cache: LayerCache, recompute_interval: int) -> Tuple[np.ndarray, np.ndarray]:
    """h/c checkpoints as the reference's forward stores them: entry k holds the state
    ENTERING step k*R (entry 0 = h0, c0); shape (ceil(T/R), B, H)
    (flashlstm_v2/src/lstm_forward.cu:727-783)."""
    T = cache.h_s.shape[0] - 1
    idx = np.arange(0, T, recompute_interval)
    return cache.h_s[idx].copy(), cache.c_s[idx].copy()


# --------------------------------------------------------------------------- metrics
def max_abs_err(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b))) if a.size else 0.0


def rel_l2_err(a, b) -> float:
    """||a-b||_2 / ||b||_2 with b the ground truth."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    den = float(np.linalg.norm(b))
    num = float(np.linalg.norm(a - b))
    return num / den if den > 0 else num
