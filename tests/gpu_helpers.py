"""Helpers for the GPU parity tests: run the engine through the C ABI on a workload and
compare with the CPU oracle / torch.nn.LSTM."""
from __future__ import annotations

import numpy as np
import torch

from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine
from oracle import lstm_oracle as orc
from tests.helpers import params_from_inputs, to_np


def run_engine(w, inp, backend="auto", dhn=None, dcn=None, repeat=1):
    """Forward (+ backward when inp.dy is given) on cuda:0.  Returns (dict of numpy arrays, engine)."""
    dev = torch.device("cuda", 0)
    td = TORCH_DTYPES[w.dtype]
    eng = Engine(w.dtype, w.layers, w.batch, w.input_size, w.hidden_size, w.seq_len, training=w.training,
                 backend=backend, device=dev)
    for l in range(w.layers):
        eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
    x = inp.x.to(dev, td)
    h0 = None if inp.h0 is None else inp.h0.to(dev, td)
    c0 = None if inp.c0 is None else inp.c0.to(dev, td)
    out = {}
    for _ in range(repeat):
        y, hn, cn = eng.forward(x, h0, c0)
        out.update(y=to_np(y), hn=to_np(hn), cn=to_np(cn))
        if inp.dy is not None:
            dx, dh0, dc0 = eng.backward(inp.dy.to(dev, td), None if dhn is None else dhn.to(dev, td),
                                        None if dcn is None else dcn.to(dev, td))
            out.update(dx=to_np(dx), dh0=to_np(dh0), dc0=to_np(dc0))
            out["dw_ih"], out["dw_hh"], out["db"] = [], [], []
            for l in range(w.layers):
                a, b, c = eng.grads(l)
                out["dw_ih"].append(to_np(a))
                out["dw_hh"].append(to_np(b))
                out["db"].append(to_np(c))
    torch.cuda.synchronize()
    return out, eng


def run_oracle(inp, dhn=None, dcn=None, dtype=np.float32):
    params = params_from_inputs(inp)
    fwd = orc.lstm_forward(inp.x.numpy(), params, None if inp.h0 is None else inp.h0.numpy(),
                           None if inp.c0 is None else inp.c0.numpy(), dtype=dtype)
    out = {"y": fwd.y, "hn": fwd.h_n, "cn": fwd.c_n, "gates": [c.gates for c in fwd.caches]}
    if inp.dy is not None:
        bwd = orc.lstm_backward(fwd, params, inp.dy.numpy(), None if dhn is None else dhn.numpy(),
                                None if dcn is None else dcn.numpy(), dtype=dtype)
        out.update(dx=bwd.dx, dh0=bwd.dh0, dc0=bwd.dc0, dw_ih=bwd.dw_ih, dw_hh=bwd.dw_hh, db=bwd.db_ih)
    return out


def assert_parity(got, ref, dtype, keys=None, fp32_max_abs=2e-3, rel_l2=1e-2):
    """The stated bar: max-abs <= 2e-3 for fp32 configurations, relative-L2 <= 1e-2 for 16-bit ones."""
    keys = keys or [k for k in ("y", "hn", "cn", "dx", "dh0", "dc0", "dw_ih", "dw_hh", "db") if k in got and k in ref]
    report = {}
    for k in keys:
        a, b = got[k], ref[k]
        pairs = list(zip(a, b)) if isinstance(a, list) else [(a, b)]
        for i, (x, y) in enumerate(pairs):
            name = f"{k}[{i}]" if isinstance(a, list) else k
            assert np.all(np.isfinite(x)), f"{name} has non-finite values"
            if dtype == "f32":
                err = orc.max_abs_err(x, y)
                report[name] = err
                assert err <= fp32_max_abs, f"{name}: max-abs {err:.3e} > {fp32_max_abs}"
            else:
                err = orc.rel_l2_err(x, y)
                report[name] = err
                assert err <= rel_l2, f"{name}: rel-L2 {err:.3e} > {rel_l2}"
    return report
