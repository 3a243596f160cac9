"""Batch-sharded data parallelism: one process per GPU, sequences split across ranks, weights
replicated, weight gradients summed with one allreduce per layer inside the engine's backward.
`torch.distributed` is used only to hand the 128-byte communicator id from rank 0 to the others."""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def exchange_unique_id(make_id: Callable[[], bytes], group=None) -> bytes:
    """Rank 0 creates the id, every rank returns the same 128 bytes.  Works on any backend
    (the payload travels as a CPU uint8 tensor on gloo, a CUDA one on nccl)."""
    rank = dist.get_rank(group)
    backend = dist.get_backend(group)
    device = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    if rank == 0:
        raw = make_id()
        if len(raw) != 128:
            raise ValueError("communicator id must be 128 bytes")
        buf = torch.tensor(list(raw), dtype=torch.uint8, device=device)
    else:
        buf = torch.zeros(128, dtype=torch.uint8, device=device)
    dist.broadcast(buf, src=0, group=group)
    return bytes(buf.cpu().tolist())


def shard_range(batch: int, rank: int, world: int):
    """Rows [lo, hi) of the global batch owned by `rank`; the batch must divide evenly."""
    if batch % world:
        raise ValueError(f"global batch {batch} is not divisible by world size {world}")
    per = batch // world
    return rank * per, (rank + 1) * per


def attach_data_parallel(target, group=None) -> None:
    """Give `target` (an Engine or an LSTM module) a communicator spanning the process group."""
    from .engine import Engine

    uid = exchange_unique_id(Engine.new_unique_id, group)
    target.attach_comm(uid, dist.get_rank(group), dist.get_world_size(group))
