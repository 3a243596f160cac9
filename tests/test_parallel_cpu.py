"""Host-side logic of the batch-sharded data-parallel path on CPU ranks (gloo, world size 2):
the communicator id reaches every rank, and summing per-shard weight gradients over ranks equals
the full-batch gradient (the identity the in-backward allreduce relies on)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashlstm_poc_b200.parallel import (ParallelSetupError, StepTimeout, StepWatchdog, check_same_config,
                                         exchange_unique_id, init_group, shard_range)
from flashlstm_poc_b200.workloads import Workload, make_inputs, shard_batch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # 1. id exchange: only rank 0's generator may run; every rank ends with the same 128 bytes
        def make_id():
            assert dist.get_rank() == 0
            return bytes((7 * i + 3) % 256 for i in range(128))

        uid = exchange_unique_id(make_id)
        # 2. shard-and-sum identity with the CPU oracle standing in for the engine
        from oracle import lstm_oracle as orc

        w = Workload("dp", "f32", 2, 12, 8, 6, 5, seed=21, state_std=0.4)
        inp = make_inputs(w)
        params = [orc.LayerParams(inp.w_ih[l].numpy(), inp.w_hh[l].numpy(), inp.b_ih[l].numpy(), inp.b_hh[l].numpy())
                  for l in range(w.layers)]
        lo, hi = shard_range(w.batch, rank, world)
        sx, sdy = shard_batch(inp.x, rank, world), shard_batch(inp.dy, rank, world)
        sh0, sc0 = shard_batch(inp.h0, rank, world), shard_batch(inp.c0, rank, world)
        assert sx.shape[1] == hi - lo and torch.equal(sx, inp.x[:, lo:hi])
        fwd = orc.lstm_forward(sx.numpy(), params, sh0.numpy(), sc0.numpy(), dtype=np.float64)
        bwd = orc.lstm_backward(fwd, params, sdy.numpy(), dtype=np.float64)
        flat = torch.from_numpy(np.concatenate([np.concatenate([bwd.dw_ih[l].ravel(), bwd.dw_hh[l].ravel(), bwd.db_ih[l]])
                                                for l in range(w.layers)]))
        dist.all_reduce(flat)  # what ncclAllReduce does to the flat [dW_ih | dW_hh | db] buffer
        full_f = orc.lstm_forward(inp.x.numpy(), params, inp.h0.numpy(), inp.c0.numpy(), dtype=np.float64)
        full_b = orc.lstm_backward(full_f, params, inp.dy.numpy(), dtype=np.float64)
        want = np.concatenate([np.concatenate([full_b.dw_ih[l].ravel(), full_b.dw_hh[l].ravel(), full_b.db_ih[l]])
                               for l in range(w.layers)])
        results[rank] = (uid, float(np.max(np.abs(flat.numpy() - want))),
                         float(np.max(np.abs(bwd.dx - full_b.dx[:, lo:hi]))))
    finally:
        dist.destroy_process_group()


def test_world_size_two_gloo():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == world
        ids = {results[r][0] for r in range(world)}
        assert len(ids) == 1 and len(next(iter(ids))) == 128
        for r in range(world):
            assert results[r][1] < 1e-10  # summed shard gradients == full-batch gradients
            assert results[r][2] < 1e-12  # dX of a shard does not depend on the other shard


def test_shard_range_rejects_uneven_batches():
    assert shard_range(64, 1, 2) == (32, 64)
    with pytest.raises(ValueError):
        shard_range(10, 0, 4)


# ---------------------------------------------------------------- failures, injected on the host only
def _failing_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    init_group("gloo", rank, world, timeout_s=60)
    out = {}
    try:
        # a. rank 0 cannot produce a valid id: every rank must raise, none may hang in the broadcast
        try:
            exchange_unique_id(lambda: b"too short")
            out["bad_id"] = "no error"
        except ParallelSetupError as exc:
            out["bad_id"] = str(exc)
        # b. the id generator itself fails on rank 0
        def broken():
            raise RuntimeError("no NCCL here")
        try:
            exchange_unique_id(broken)
            out["broken_id"] = "no error"
        except ParallelSetupError as exc:
            out["broken_id"] = str(exc)
        # c. engines built with different shapes on the two ranks
        try:
            check_same_config(("f16", 1, 32, 1024, 1024 if rank == 0 else 2048, True))
            out["mismatch"] = "no error"
        except ParallelSetupError as exc:
            out["mismatch"] = str(exc)
        # d. and the agreeing case passes, after the failures, on the same group
        check_same_config(("f16", 1, 32, 1024, 1024, True))
        out["uid_len"] = len(exchange_unique_id(lambda: bytes(range(128))))
    finally:
        dist.destroy_process_group()
    results[rank] = out


def test_setup_failures_are_raised_on_every_rank():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_failing_worker, args=(world, port, results), nprocs=world, join=True)
        for r in range(world):
            out = results[r]
            assert "128-byte" in out["bad_id"] and "128-byte" in out["broken_id"]
            assert "rank 1 has" in out["mismatch"] and "2048" in out["mismatch"]
            assert out["uid_len"] == 128


def _lonely_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    try:
        init_group("gloo", rank, world, timeout_s=3)
        results[rank] = "joined"
        dist.destroy_process_group()
    except ParallelSetupError as exc:
        results[rank] = str(exc)


def test_a_rank_that_never_joins_ends_setup_with_an_error():
    """World size 2, but only rank 0 is started (its peer died before start-up)."""
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_lonely_worker, args=(2, port, results), nprocs=1, join=True)
        assert "did not form within 3 s" in results[0]


def test_step_watchdog_policy():
    """The deadline policy with a fake clock: a step that finishes is left alone; one that does not gets its
    communicator aborted exactly once and the caller an exception."""
    now = [0.0]
    clock = lambda: now[0]
    def sleep(dt):
        now[0] += dt
    polls = [0]
    def done_after_5():
        polls[0] += 1
        return polls[0] > 5
    aborted = []
    wd = StepWatchdog(1.0, done_after_5, lambda: aborted.append(1), clock=clock, sleep=sleep, poll_s=0.01)
    assert wd.wait() == pytest.approx(0.05) and not aborted and not wd.aborted
    wd = StepWatchdog(0.25, lambda: False, lambda: aborted.append(1), clock=clock, sleep=sleep, poll_s=0.01)
    with pytest.raises(StepTimeout, match="0.25 s"):
        wd.wait()
    assert aborted == [1] and wd.aborted
