"""Host-side plumbing for running one replica per GPU: which rows a rank owns, the max-over-ranks
reduction used for timing, and the final gather of per-rank outputs on the host.

The forward path itself has no exchange step: samples / rows are independent, every rank holds a
full replica and processes its own slice.  torch.distributed is used for the barrier and these small
host-side reductions only (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

import numpy as np


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous slice [begin, end) of `total` units for `rank`; the first `total % world` ranks
    take one extra unit.  Slices are disjoint and cover everything."""
    import ctypes as C

    from . import runtime as rt

    b, e = C.c_longlong(), C.c_longlong()
    if rt.lib().mimir_b200_shard_range(total, world, rank, C.byref(b), C.byref(e)) != 0:  # the library's own slicing rule
        raise ValueError("bad shard arguments")
    return b.value, e.value


def reduce_max(value: float, device=None) -> float:
    """Max of a per-rank scalar over all ranks (identity without an initialised process group)."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_rows(local: np.ndarray, total_rows: int, dst: int = 0):
    """Final host gather: every rank passes the rows it computed (its shard_range slice, in order);
    rank `dst` gets the full [total_rows, ...] array, the others None."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        if local.shape[0] != total_rows:
            raise ValueError("single rank must hold every row")
        return local
    world, rank = dist.get_world_size(), dist.get_rank()
    b, e = shard_range(total_rows, world, rank)
    if local.shape[0] != e - b:
        raise ValueError(f"rank {rank} holds {local.shape[0]} rows, its shard is {e - b}")
    parts = [None] * world if rank == dst else None
    dist.gather_object(local, parts, dst=dst)
    if rank != dst:
        return None
    return np.concatenate(parts, axis=0)
