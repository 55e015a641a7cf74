"""Host-side sharding plans for the multi-GPU paths (one process per GPU).

* ranking requests are independent -> data parallel: `split_batch`;
* the unified embedding table and the retrieval corpus are row-sharded in contiguous ranges, the ownership rule of
  the reference (phoenix/xrex/cuda/row_emb/src/row_emb_kernel.hpp:19-25: owner = row / rows_per_rank;
  phoenix/xrex/models/recsys_two_tower_model.py:216: global row = shard * rows_local + local);
* `attach_table_shards` wires the engines of a torch.distributed job together: every rank exports its table shard
  as a CUDA IPC handle, all-gathers the handles and maps the other ranks' shards, after which the gather kernel
  reads remote rows over NVLink directly (no id / row exchange collectives on the data path);
* `ShardedGatherSum` is the reference's exchange itself (phoenix/xrex/cuda/row_emb/src/row_emb_comm.cc:655-743):
  row requests grouped by owner, NCCL all-to-all of the row numbers, owner-side gather, NCCL all-to-all of the rows,
  fixed-order sum at the requester.  Bulk transfers reach several times the NVLink throughput of the per-row peer
  loads, so this is the path for large id batches; both give bit-identical results.
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


class ShardedGatherSum:
    """Multi-hash gather-sum over a table row-sharded across the ranks of a torch.distributed (NCCL) group.

    `engine` holds this rank's shard (`PhoenixConfig(table_world=W, table_rank=r)`); each call takes this rank's ids
    and returns their summed rows, like `engine.gather_sum_device` on an unsharded table, bit for bit.  All kernels
    and collectives run on the current torch CUDA stream; the only host synchronisation is the read of the two count
    vectors that size the variable all-to-all."""

    def __init__(self, engine, max_ids: int, group=None):
        import torch
        import torch.distributed as dist
        self.eng, self.group = engine, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        cfg = engine.cfg
        assert cfg.table_world == self.world and cfg.table_rank == self.rank
        self.H, self.width = cfg.num_hashes, cfg.emb_size
        self.shard_rows = rows_per_shard(cfg.table_rows, self.world)
        dev = torch.device("cuda", torch.cuda.current_device())
        nreq = max_ids * self.H
        i32 = dict(dtype=torch.int32, device=dev)
        self.rows = torch.empty(nreq, **i32)
        self.send_rows = torch.empty(nreq, **i32)
        self.pos = torch.empty(nreq, **i32)
        self.counts = torch.empty(self.world, **i32)
        self.cursor = torch.empty(self.world, **i32)
        self.recv_counts = torch.empty(self.world, **i32)
        self.back = torch.empty((nreq, self.width), dtype=torch.int16, device=dev)
        self._recv_rows = torch.empty(0, **i32)
        self._gathered = torch.empty((0, self.width), dtype=torch.int16, device=dev)
        self.max_ids = max_ids

    def __call__(self, family: int, ids, n: int, out):
        import torch
        import torch.distributed as dist
        from . import _lib
        from .engine import _ptr
        lib = _lib.lib
        assert n <= self.max_ids
        st = torch.cuda.current_stream().cuda_stream
        nreq = n * self.H

        def chk(status):
            if status != 0:
                raise _lib.PhoenixError(status, lib.phx_global_error().decode())

        # ids -> unified-table rows (engine stream), then everything else on torch's stream
        self.eng.hash_ids_device(family, ids, n, self.rows)
        self.eng.sync()
        chk(lib.phx_shard_bucket(_ptr(self.rows), nreq, self.shard_rows, self.world, _ptr(self.counts), _ptr(self.cursor),
                                 _ptr(self.send_rows), _ptr(self.pos), st))
        dist.all_to_all_single(self.recv_counts, self.counts, group=self.group)
        send_splits = self.counts.tolist()            # host sync: the variable all-to-all needs its sizes
        recv_splits = self.recv_counts.tolist()
        m = sum(recv_splits)
        if self._recv_rows.numel() < m:               # grows to the largest request volume seen, then stays
            self._recv_rows = torch.empty(int(m * 1.25) + 1, dtype=torch.int32, device=self.rows.device)
            self._gathered = torch.empty((int(m * 1.25) + 1, self.width), dtype=torch.int16, device=self.rows.device)
        recv_rows, gathered = self._recv_rows[:m], self._gathered[:m]
        dist.all_to_all_single(recv_rows, self.send_rows[:nreq], recv_splits, send_splits, group=self.group)
        chk(lib.phx_shard_gather_rows(self.eng.table_local_ptr(), self.shard_rows, _ptr(recv_rows), m, self.width,
                                      _ptr(gathered), st))
        back = self.back[:nreq]
        dist.all_to_all_single(back, gathered, send_splits, recv_splits, group=self.group)
        chk(lib.phx_shard_sum_rows(_ptr(back), _ptr(self.pos), n, self.H, self.width, _ptr(out), st))
        return out
