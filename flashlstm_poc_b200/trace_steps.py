"""Per-time-step clock trace of the persistent recurrent kernels (tensor-core backend).

    python -m flashlstm_poc_b200.trace_steps [workload-name]

CTA 0 of the forward and of the BPTT kernel stamps clock64() at fixed points of each of the first 64
time steps (flstm_engine_enable_trace); this prints, per point, the median distance in SM cycles from
the previous step's release, i.e. where a step's time goes."""
import ctypes
import sys

import numpy as np
import torch

from flashlstm_poc_b200.engine import Engine
from flashlstm_poc_b200.workloads import WORKLOADS, make_inputs
w = WORKLOADS[sys.argv[1] if len(sys.argv) > 1 else 'c2_fp16_h1024']; inp = make_inputs(w); dev = torch.device('cuda',0)
eng = Engine(w.dtype, 1, w.batch, w.input_size, w.hidden_size, w.seq_len, device=dev)
eng.set_weights(0, inp.w_ih[0].to(dev), inp.w_hh[0].to(dev), inp.b_ih[0].to(dev), inp.b_hh[0].to(dev))
x = inp.x.to(dev, torch.float16); dy = inp.dy.to(dev, torch.float16)
h0 = inp.h0.to(dev, torch.float16); c0 = inp.c0.to(dev, torch.float16)
for _ in range(3):
    eng.forward(x,h0,c0); eng.backward(dy)
N = 64
assert eng.lib.flstm_engine_enable_trace(eng._h, N) == 0
eng.forward(x,h0,c0); eng.backward(dy); torch.cuda.synchronize()
buf = (ctypes.c_longlong * (2*N*16))()
assert eng.lib.flstm_engine_read_trace(eng._h, buf, 2*N*16) == 0
a = np.array(buf[:], dtype=np.int64).reshape(2, N, 16)
names = {0:'barrier seen',1:'tma issued',2:'first chunk',3:'last chunk',4:'mma committed',5:'tfull seen',9:'partials sent / proxy fence done',10:'reduce ready',6:'after exchange',7:'stores issued',8:'released'}
for d, nm in ((0,'FWD'),(1,'BWD')):
    t = a[d]
    print(nm, 'step period (clk) median:', np.median(np.diff(t[8:60,8])))
    base = t[10:60, 8][:-1]   # release of previous step
    for k in ((0,1,2,3,4,5,6,7,9,8) if d == 0 else (0,1,2,3,4,5,9,10,6,7,8)):
        v = t[11:60, k] - base
        if t[11:60,k].min() == 0: continue
        print(f'  {names[k]:>16}: median {np.median(v):8.0f} clk  min {v.min():8.0f} max {v.max():8.0f}')
