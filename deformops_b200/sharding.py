"""Batch sharding of the MSDA path over the GPUs of one box.

Every output row and every gradient of the operator depends on its own batch element only
(the reference already splits the batch on the host,
``sources/deformops/backends/cuda/include/msda_launch.cuh:107-131``), so ranks take
contiguous batch slices and never exchange tensor data.  ``torch.distributed`` is used for
two host-side things only: aligning the start of a timed region and taking the maximum of
the per-rank device times.
"""

from __future__ import annotations

import dataclasses
import os

import torch

__all__ = ["Shard", "init_from_env", "shard_batch", "max_over_ranks", "barrier"]


@dataclasses.dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    first_sample: int   # global index of this rank's first sample
    batch: int          # samples held by this rank


def shard_batch(global_batch: int, world: int, rank: int) -> Shard:
    """Contiguous, near-even split: the first ``global_batch % world`` ranks get one more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in [0, {world})")
    if global_batch < 0:
        raise ValueError("global_batch must be >= 0")
    base, extra = divmod(global_batch, world)
    batch = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return Shard(rank=rank, world=world, first_sample=first, batch=batch)


def init_from_env(backend: str | None = None, device: "torch.device | None" = None) -> tuple[int, int, int]:
    """Join the process group torchrun describes; returns ``(rank, world, local_rank)``.

    A single process (no ``WORLD_SIZE`` or ``WORLD_SIZE=1``) joins nothing.
    """
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not torch.distributed.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs = {"device_id": device} if (backend == "nccl" and device is not None) else {}
        torch.distributed.init_process_group(backend, **kwargs)
    return rank, world, local_rank


def barrier() -> None:
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def max_over_ranks(values: list[float], device="cpu") -> list[float]:
    """Element-wise maximum of per-rank numbers (device times) over all ranks."""
    t = torch.tensor(values, dtype=torch.float64, device=device)
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return t.tolist()
