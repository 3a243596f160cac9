"""One process driving engines on two GPUs: the opt-in shared-memory limit of a kernel is a per-device
attribute, and every entry point must work on the engine's own device whatever device is current."""
import pytest
import torch

from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine
from flashlstm_poc_b200.workloads import Workload, make_inputs
from tests.gpu_helpers import assert_parity, run_oracle
from tests.helpers import to_np

pytestmark = pytest.mark.gpu


def _run(eng, w, inp, dev):
    td = TORCH_DTYPES[w.dtype]
    y, hn, cn = eng.forward(inp.x.to(dev, td))
    dx, dh0, dc0 = eng.backward(inp.dy.to(dev, td))
    torch.cuda.synchronize(dev)
    out = dict(y=to_np(y), hn=to_np(hn), cn=to_np(cn), dx=to_np(dx), dh0=to_np(dh0), dc0=to_np(dc0))
    out["dw_ih"], out["dw_hh"], out["db"] = map(list, zip(*[[to_np(g) for g in eng.grads(l)] for l in range(w.layers)]))
    return out


@pytest.mark.parametrize("dtype,hidden,batch", [("bf16", 256, 32), ("f16", 1024, 96), ("f32", 128, 16)])
def test_engines_on_two_devices_in_one_process(dtype, hidden, batch):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    w = Workload("two-dev", dtype, 2, 128, hidden, batch, 6, seed=5)
    inp = make_inputs(w)
    ref = run_oracle(inp)
    devs = [torch.device("cuda", 0), torch.device("cuda", 1)]
    engines = []
    for dev in devs:
        eng = Engine(w.dtype, w.layers, w.batch, w.input_size, w.hidden_size, w.seq_len, device=dev)
        for l in range(w.layers):
            eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
        engines.append(eng)
    torch.cuda.set_device(0)  # the second engine is driven while another device is current
    results = [_run(eng, w, inp, dev) for eng, dev in zip(engines, devs)]
    assert torch.cuda.current_device() == 0
    for eng in engines:
        eng.close()
    for got in results:
        assert_parity(got, ref, w.dtype)
