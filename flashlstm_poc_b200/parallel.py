"""Batch-sharded data parallelism: one process per GPU, sequences split across ranks, weights
replicated, weight gradients summed with one allreduce per layer inside the engine's backward.
`torch.distributed` is used only for the host-side plumbing: handing the 128-byte communicator id
from rank 0 to the others and checking that every rank built the same engine.

Failure handling lives on the host as well.  Setup errors (a bad id, engines that differ between
ranks) are raised on EVERY rank, so no rank is left waiting in a collective the others never enter.
A step that does not finish by its deadline is given up by `StepWatchdog`: it aborts the
communicator (so a collective a lost peer will never join cannot block the process) and raises."""

from __future__ import annotations

import time
from typing import Callable, Optional

import torch
import torch.distributed as dist


class ParallelSetupError(ValueError):
    """The ranks of a data-parallel group do not agree (raised on every rank)."""


class StepTimeout(RuntimeError):
    """A step missed its deadline; the communicator has been aborted."""


def _plumbing_device(group) -> torch.device:
    backend = dist.get_backend(group)
    return torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")


def init_group(backend: str, rank: int, world_size: int, timeout_s: float = 600.0, **kwargs) -> None:
    """`torch.distributed.init_process_group` with a deadline: a rank that never shows up (died before
    start-up, wrong address) turns into ParallelSetupError on the ranks that did, instead of an open-ended wait."""
    import datetime

    try:
        dist.init_process_group(backend, rank=rank, world_size=world_size,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    except Exception as exc:  # DistStoreError / DistNetworkError / RuntimeError depending on where it stalls
        raise ParallelSetupError(f"rank {rank}: process group of {world_size} did not form within {timeout_s:g} s: {exc}") from exc


def exchange_unique_id(make_id: Callable[[], bytes], group=None) -> bytes:
    """Rank 0 creates the id, every rank returns the same 128 bytes.  Works on any backend
    (the payload travels as a CPU uint8 tensor on gloo, a CUDA one on nccl).  If rank 0 cannot
    produce a valid id, every rank raises ParallelSetupError (a flag byte travels with the id)."""
    rank = dist.get_rank(group)
    device = _plumbing_device(group)
    payload = torch.zeros(129, dtype=torch.uint8, device=device)
    if rank == 0:
        try:
            raw = make_id()
            ok = isinstance(raw, (bytes, bytearray)) and len(raw) == 128
        except Exception:  # the failure is reported to every rank below
            raw, ok = b"", False
        if ok:
            payload = torch.tensor([1] + list(raw), dtype=torch.uint8, device=device)
    dist.broadcast(payload, src=0, group=group)
    got = bytes(payload.cpu().tolist())
    if got[0] != 1:
        raise ParallelSetupError("rank 0 could not create a 128-byte communicator id")
    return got[1:]


def check_same_config(config: tuple, group=None) -> None:
    """Every rank passes what it built its engine with; a disagreement raises ParallelSetupError on all
    ranks, naming the ranks that differ from rank 0 (mismatched shapes would otherwise surface as a hung
    or corrupt allreduce)."""
    world = dist.get_world_size(group)
    configs = [None] * world
    dist.all_gather_object(configs, tuple(config), group=group)
    bad = [r for r in range(world) if configs[r] != configs[0]]
    if bad:
        raise ParallelSetupError(
            f"engine configuration differs between ranks: rank 0 has {configs[0]}, "
            + ", ".join(f"rank {r} has {configs[r]}" for r in bad))


def shard_range(batch: int, rank: int, world: int):
    """Rows [lo, hi) of the global batch owned by `rank`; the batch must divide evenly."""
    if batch % world:
        raise ValueError(f"global batch {batch} is not divisible by world size {world}")
    per = batch // world
    return rank * per, (rank + 1) * per


def attach_data_parallel(target, group=None) -> None:
    """Give `target` (an Engine or an LSTM module) a communicator spanning the process group."""
    from .engine import Engine

    engine = getattr(target, "engine", target)
    key = getattr(engine, "config_key", None)
    if key is not None:
        check_same_config(key, group)
    uid = exchange_unique_id(Engine.new_unique_id, group)
    target.attach_comm(uid, dist.get_rank(group), dist.get_world_size(group))


class StepWatchdog:
    """Deadline for one step.  `query()` says whether the step's device work has finished, `abort()` gives
    the communicator up.  With an engine, `StepWatchdog.for_engine(engine, deadline_s).wait()` is
    `engine.wait(deadline_s)` (the polling happens in the library); the callable form exists so the policy
    can be exercised without a GPU."""

    def __init__(self, deadline_s: float, query: Callable[[], bool], abort: Callable[[], None],
                 clock: Callable[[], float] = time.monotonic, sleep: Callable[[float], None] = time.sleep,
                 poll_s: float = 1e-3):
        self.deadline_s, self.query, self.abort = float(deadline_s), query, abort
        self.clock, self.sleep, self.poll_s = clock, sleep, poll_s
        self.aborted = False

    @classmethod
    def for_engine(cls, engine, deadline_s: float, stream: Optional[torch.cuda.Stream] = None) -> "StepWatchdog":
        done = torch.cuda.Event()
        done.record(stream if stream is not None else torch.cuda.current_stream())
        return cls(deadline_s, done.query, engine.abort_comm)

    def wait(self) -> float:
        """Returns the seconds waited; raises StepTimeout after aborting when the deadline passes."""
        start = self.clock()
        while True:
            if self.query():
                return self.clock() - start
            if self.clock() - start >= self.deadline_s:
                self.aborted = True
                self.abort()
                raise StepTimeout(f"step did not finish within {self.deadline_s:g} s; communicator aborted")
            self.sleep(self.poll_s)
