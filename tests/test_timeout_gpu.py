"""The bounded-wait exit path of the persistent kernels, exercised without faulting, trapping or hanging anything.

The host asks the step barrier to wait for one arrival more than the CTAs of a batch group make
(flstm_engine_selftest_missing_arrivals) and shortens the limit of every device-side wait to a few
milliseconds (flstm_engine_set_wait_limit).  The wait of the second time step then runs out: the kernel raises
its error word, every role drains and the launch RETURNS; the host sees FLSTM_ERR_TIMEOUT, and the same engine
then computes a normal step whose results are bit-identical to the ones it produced before."""
import time

import numpy as np
import pytest
import torch

from flashlstm_poc_b200._lib import FlashLstmError
from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine
from flashlstm_poc_b200.workloads import Workload, make_inputs

pytestmark = pytest.mark.gpu

LIMIT_US = 5000  # 5 ms


def _engine(w, inp, backend):
    dev = torch.device("cuda", 0)
    eng = Engine(w.dtype, w.layers, w.batch, w.input_size, w.hidden_size, w.seq_len, backend=backend, device=dev)
    for l in range(w.layers):
        eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
    return eng, dev


def _step(eng, inp, dev, td):
    y, hn, cn = eng.forward(inp.x.to(dev, td), inp.h0.to(dev, td), inp.c0.to(dev, td))
    dx, dh0, dc0 = eng.backward(inp.dy.to(dev, td))
    torch.cuda.synchronize()
    out = [y, hn, cn, dx, dh0, dc0] + [g for l in range(eng.layers) for g in eng.grads(l)]
    return [t.detach().float().cpu().numpy().copy() for t in out]


@pytest.mark.parametrize("dtype,backend,where", [
    ("f16", "tc", "forward"), ("f16", "tc", "backward"), ("bf16", "tc", "forward"),
    ("f32", "simt", "forward"), ("f32", "simt", "backward"),
    ("bf16", "tc", "forward-wide"),  # 96 sequences at H = 1024: the wide-batch forward kernel (all steps in one launch)
    # H = 2048: W_hh is streamed, and part of it is fetched into the ring ahead of the barrier that then fails
    ("bf16", "tc", "forward-streamed"), ("bf16", "tc", "backward-streamed"),
])
def test_step_barrier_timeout_returns_and_engine_recovers(dtype, backend, where):
    where, _, variant = where.partition("-")
    shape = {"": (64, 64, 8), "wide": (128, 1024, 96), "streamed": (128, 2048, 8)}[variant]
    w = Workload("timeout", dtype, 1, *shape, 4, seed=11, state_std=0.1)
    inp = make_inputs(w)
    td = TORCH_DTYPES[dtype]
    eng, dev = _engine(w, inp, backend)
    assert eng.backend == backend
    before = _step(eng, inp, dev, td)
    assert all(np.isfinite(a).all() for a in before) and np.abs(before[0]).max() <= 1.0  # every row of y was written

    eng.set_wait_limit(LIMIT_US)
    x, h0, c0, dy = (t.to(dev, td) for t in (inp.x, inp.h0, inp.c0, inp.dy))
    t_start = time.perf_counter()
    if where == "forward":
        eng.selftest_missing_arrivals(1)
        eng.forward(x, h0, c0)          # enqueued; the kernel gives up at the barrier of the second step
    else:
        eng.forward(x, h0, c0)
        eng.selftest_missing_arrivals(1)
        eng.backward(dy)
    with pytest.raises(FlashLstmError) as exc:
        eng.wait(20.0)                  # host watchdog: the launch has returned, the error word is set
    waited = time.perf_counter() - t_start
    assert exc.value.status == 3, exc.value  # FLSTM_ERR_TIMEOUT
    assert waited < 5.0, f"the kernel took {waited:.2f} s to give up with a {LIMIT_US} us limit"
    torch.cuda.synchronize()            # the context is intact

    eng.selftest_missing_arrivals(0)
    eng.set_wait_limit(0)
    after = _step(eng, inp, dev, td)
    eng.close()
    for a, b in zip(before, after):
        assert np.array_equal(a, b)
