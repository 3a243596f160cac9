"""Batch-sharded data parallelism on real GPUs (needs >= 2 devices; skipped otherwise): every rank
runs its shard through the engine, the per-layer NCCL allreduce inside backward sums the weight
gradients, and the result equals the CPU oracle's full-batch gradients."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, dtype, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flashlstm_poc_b200.engine import TORCH_DTYPES, Engine
        from flashlstm_poc_b200.parallel import attach_data_parallel
        from flashlstm_poc_b200.workloads import Workload, make_inputs, shard_batch

        w = Workload("dp", dtype, 2, 64, 64, 16 * world, 12, seed=5, state_std=0.3)
        inp = make_inputs(w)
        td = TORCH_DTYPES[dtype]
        eng = Engine(dtype, w.layers, w.batch // world, w.input_size, w.hidden_size, w.seq_len, device=dev)
        for l in range(w.layers):
            eng.set_weights(l, inp.w_ih[l].to(dev), inp.w_hh[l].to(dev), inp.b_ih[l].to(dev), inp.b_hh[l].to(dev))
        attach_data_parallel(eng)
        sh = lambda t: shard_batch(t, rank, world).to(dev, td)
        for _ in range(2):  # twice: the communicator and the event fork/join are reusable
            y, hn, cn = eng.forward(sh(inp.x), sh(inp.h0), sh(inp.c0))
            dx, dh0, dc0 = eng.backward(sh(inp.dy))
        torch.cuda.synchronize()
        grads = [[g.float().cpu().numpy() for g in eng.grads(l)] for l in range(w.layers)]
        # Giving the communicator up and starting over, BETWEEN steps (nothing in flight on any rank, every
        # rank does it: no collective is left without a peer).  A backward without communicator must refuse.
        from flashlstm_poc_b200._lib import FlashLstmError

        eng.wait(60.0)
        eng.abort_comm()
        eng.forward(sh(inp.x), sh(inp.h0), sh(inp.c0))
        try:
            eng.backward(sh(inp.dy))
            refused = False
        except FlashLstmError as exc:
            refused = "aborted" in str(exc)
        torch.cuda.synchronize()
        dist.barrier()
        attach_data_parallel(eng)
        eng.forward(sh(inp.x), sh(inp.h0), sh(inp.c0))
        eng.backward(sh(inp.dy))
        torch.cuda.synchronize()
        again = eng.grads(0)[0].float().cpu().numpy()
        results[rank] = (eng.backend, grads, dx.float().cpu().numpy(), refused, bool(np.array_equal(again, grads[0][0])))
        eng.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_two_rank_gradients_match_full_batch_oracle(dtype):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from flashlstm_poc_b200.workloads import Workload, make_inputs
    from oracle import lstm_oracle as orc
    from tests.gpu_helpers import run_oracle

    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), dtype, results), nprocs=world, join=True)
        w = Workload("dp", dtype, 2, 64, 64, 16 * world, 12, seed=5, state_std=0.3)
        ref = run_oracle(make_inputs(w))
        for r in range(world):
            backend, grads, dx, refused, same_after_reattach = results[r]
            assert backend == ("tc" if dtype == "f16" else "simt")
            assert refused and same_after_reattach
            for l in range(w.layers):
                for got, want in zip(grads[l], (ref["dw_ih"][l], ref["dw_hh"][l], ref["db"][l])):
                    err = orc.rel_l2_err(got, want)
                    assert err < (1e-2 if dtype == "f16" else 1e-5), (r, l, err)
            lo = r * 16
            assert orc.rel_l2_err(dx, ref["dx"][:, lo:lo + 16]) < (1e-2 if dtype == "f16" else 1e-5)
        # every rank holds the same reduced gradients
        assert np.array_equal(results[0][1][0][0], results[1][1][0][0])
