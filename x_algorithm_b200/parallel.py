"""Host-side sharding plans for the multi-GPU paths (one process per GPU).

* ranking requests are independent -> data parallel: `split_batch`;
* the unified embedding table and the retrieval corpus are row-sharded in contiguous ranges, the ownership rule of
  the reference (phoenix/xrex/cuda/row_emb/src/row_emb_kernel.hpp:19-25: owner = row / rows_per_rank;
  phoenix/xrex/models/recsys_two_tower_model.py:216: global row = shard * rows_local + local);
* `attach_table_shards` wires the engines of a torch.distributed job together: every rank exports its table shard
  as a CUDA IPC handle, all-gathers the handles and maps the other ranks' shards, after which the gather kernel
  reads remote rows over NVLink directly (no id / row exchange collectives on the data path).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def rows_per_shard(total_rows: int, world: int) -> int:
    return (total_rows + world - 1) // world


def shard_range(total_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """[lo, hi) of the rows rank `rank` owns."""
    rps = rows_per_shard(total_rows, world)
    lo = min(rank * rps, total_rows)
    return lo, min(lo + rps, total_rows)


def owner_of(rows: np.ndarray, total_rows: int, world: int) -> Tuple[np.ndarray, np.ndarray]:
    """(owner rank, local row) of global rows; out-of-range rows map to row 0 like the gather does."""
    rows = np.asarray(rows, dtype=np.int64)
    rows = np.where((rows < 0) | (rows >= total_rows), 0, rows)
    rps = rows_per_shard(total_rows, world)
    return rows // rps, rows % rps


def split_batch(n: int, world: int, rank: int) -> Tuple[int, int]:
    """[lo, hi) of the requests rank `rank` serves when a batch of n is split as evenly as possible."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def attach_table_shards(engine, group=None) -> None:
    """Exchange CUDA IPC handles of the table shards over torch.distributed and map the peers' shards."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    assert engine.cfg.table_world == world and engine.cfg.table_rank == rank
    handles: List[bytes] = [b""] * world
    dist.all_gather_object(handles, engine.table_ipc_handle(), group=group)
    for r, h in enumerate(handles):
        if r != rank:
            engine.table_attach_peer(r, h)
    dist.barrier(group)
