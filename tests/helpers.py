"""Shared helpers for the test-suite: ground truth via torch.nn.LSTM and the oracle."""
from __future__ import annotations

import glob
import os

import numpy as np
import torch

from oracle import lstm_oracle as orc

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_cases():
    return sorted(glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def params_from_inputs(inp):
    return [
        orc.LayerParams(inp.w_ih[l].numpy(), inp.w_hh[l].numpy(), inp.b_ih[l].numpy(), inp.b_hh[l].numpy())
        for l in range(len(inp.w_ih))
    ]


def torch_lstm_reference(inp, dhn=None, dcn=None, dtype=torch.float32):
    """fp32 (or fp64) CPU torch.nn.LSTM forward + autograd with loss = sum(y*dY) (+ state terms).

    Returns a dict of numpy arrays: y, hn, cn and, when inp.dy is given, dx, dh0, dc0,
    dw_ih[l], dw_hh[l], db_ih[l], db_hh[l]."""
    L = len(inp.w_ih)
    I = inp.w_ih[0].shape[1]
    H = inp.w_hh[0].shape[1]
    T, B, _ = inp.x.shape
    m = torch.nn.LSTM(I, H, num_layers=L).to(dtype)
    with torch.no_grad():
        for l in range(L):
            getattr(m, f"weight_ih_l{l}").copy_(inp.w_ih[l])
            getattr(m, f"weight_hh_l{l}").copy_(inp.w_hh[l])
            getattr(m, f"bias_ih_l{l}").copy_(inp.b_ih[l])
            getattr(m, f"bias_hh_l{l}").copy_(inp.b_hh[l])
    x = inp.x.to(dtype).clone().requires_grad_(inp.dy is not None)
    h0 = (torch.zeros(L, B, H) if inp.h0 is None else inp.h0).to(dtype).clone().requires_grad_(inp.dy is not None)
    c0 = (torch.zeros(L, B, H) if inp.c0 is None else inp.c0).to(dtype).clone().requires_grad_(inp.dy is not None)
    y, (hn, cn) = m(x, (h0, c0))
    out = {"y": y.detach().numpy(), "hn": hn.detach().numpy(), "cn": cn.detach().numpy()}
    if inp.dy is not None:
        loss = (y * inp.dy.to(dtype)).sum()
        if dhn is not None:
            loss = loss + (hn * dhn.to(dtype)).sum()
        if dcn is not None:
            loss = loss + (cn * dcn.to(dtype)).sum()
        loss.backward()
        out.update(dx=x.grad.numpy(), dh0=h0.grad.numpy(), dc0=c0.grad.numpy())
        for k in ("weight_ih", "weight_hh", "bias_ih", "bias_hh"):
            out["d" + k.replace("weight", "w").replace("bias", "b")] = [
                getattr(m, f"{k}_l{l}").grad.numpy() for l in range(L)
            ]
    return out


def to_np(t):
    return t.detach().float().cpu().numpy()
