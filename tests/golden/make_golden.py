"""Generate golden vectors by RUNNING the reference's own CPU code for this path.

The reference keeps a pure-PyTorch restatement of its LSTM forward/backward in
flashlstm_v2/playground/simple_lstm_bwd.py (create_lstm_handle, lstm_forward,
lstm_backward_cudnn_like).  This script imports that file from a checkout of the
reference, runs it on seeded inputs and stores inputs + outputs as .npz fixtures next to
this file.  The fixtures travel with the repository; the reference checkout does not.

usage: python tests/golden/make_golden.py <path-to-reference-checkout>
"""

from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, T, B, I, H, seed, state_std); shapes follow the reference's own tests:
# playground (5,3,4,6); pytest (4,2,3,5); validate scripts (16,8,64,32), (32,4,128,16)
CASES = [
    ("playground_t5_b3_i4_h6", 5, 3, 4, 6, 0, 1.0),
    ("pytest_t4_b2_i3_h5", 4, 2, 3, 5, 1234, 1.0),
    ("validate_t16_b8_i64_h32", 16, 8, 64, 32, 42, 1.0),
    ("validate_t32_b4_i128_h16", 32, 4, 128, 16, 43, 0.0),
    ("single_step_t1_b1_i4_h4", 1, 1, 4, 4, 7, 1.0),
]


def load_reference(root: str):
    path = os.path.join(root, "flashlstm_v2", "playground", "simple_lstm_bwd.py")
    spec = importlib.util.spec_from_file_location("ref_simple_lstm_bwd", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod  # dataclasses resolve annotations through sys.modules
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    root = sys.argv[1]
    ref = load_reference(root)
    for name, T, B, I, H, seed, state_std in CASES:
        g = torch.Generator().manual_seed(seed)
        k = 1.0 / np.sqrt(H)
        w_ih = (torch.rand(4 * H, I, generator=g) * 2 - 1) * k
        w_hh = (torch.rand(4 * H, H, generator=g) * 2 - 1) * k
        b_ih = (torch.rand(4 * H, generator=g) * 2 - 1) * k
        b_hh = (torch.rand(4 * H, generator=g) * 2 - 1) * k
        x = torch.randn(T, B, I, generator=g)
        h0 = torch.randn(1, B, H, generator=g) * state_std
        c0 = torch.randn(1, B, H, generator=g) * state_std
        dy = torch.randn(T, B, H, generator=g)
        dhn = torch.randn(1, B, H, generator=g)
        dcn = torch.randn(1, B, H, generator=g)

        handle = ref.create_lstm_handle(w_ih, w_hh, b_ih, b_hh)
        y, (hn, cn), cache = ref.lstm_forward(handle, x, h0, c0, return_cache=True)
        dx, dw_ih, dw_hh, db_ih, db_hh, dh0, dc0 = ref.lstm_backward_cudnn_like(dy, cache, dhn, dcn)
        gates = torch.cat([cache["i_s"], cache["f_s"], cache["g_s"], cache["o_s"]], dim=2)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            w_ih=w_ih.numpy(), w_hh=w_hh.numpy(), b_ih=b_ih.numpy(), b_hh=b_hh.numpy(),
            x=x.numpy(), h0=h0.numpy(), c0=c0.numpy(), dy=dy.numpy(), dhn=dhn.numpy(), dcn=dcn.numpy(),
            y=y.numpy(), hn=hn.numpy(), cn=cn.numpy(),
            h_s=cache["h_s"].numpy(), c_s=cache["c_s"].numpy(), gates=gates.numpy(),
            dx=dx.numpy(), dw_ih=dw_ih.numpy(), dw_hh=dw_hh.numpy(),
            db_ih=db_ih.numpy(), db_hh=db_hh.numpy(), dh0=dh0.numpy(), dc0=dc0.numpy(),
        )
        print("wrote", name)


if __name__ == "__main__":
    main()
