"""world_size-2 gloo tests (CPU) of the multi-GPU plans: row-sharded gather with an id / row exchange, sharded
top-k with all-gather + merge, data-parallel batch split.  The arithmetic is the oracle's; what is under test is the
sharding plan (who owns which row, how partial results recombine) that the GPU path uses with NVLink loads / NCCL."""
import math
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import phoenix_oracle as po
        from x_algorithm_b200 import parallel as pl
        # ---- row-sharded gather-sum: ids -> rows -> owners; ids out, rows back; fixed-order sum ---------------
        cfg = po.ModelConfig(emb_size=64, num_hashes=4, table_size=1 << 10)
        lay = cfg.hash_layout()
        total = lay.total_rows
        lo, hi = pl.shard_range(total, world, rank)
        my_rows = po.synthetic_table_rows(np.arange(lo, hi), 64, 9, 0.1)            # this rank's shard only
        ids = po.make_batch(cfg, 8, seed=100 + rank, zipf_s=1.1).cand_post_ids.ravel()
        ids[:2] = [0, -3]
        rows = lay.item_hash(ids)                                                   # [n, 4] global rows
        owner, local = pl.owner_of(rows.ravel(), total, world)
        send = [torch.from_numpy(local[owner == r].copy()) for r in range(world)]
        def all_to_all(parts):   # gloo has no all-to-all: every rank publishes its parts, takes what is addressed to it
            everyone = [None] * world
            dist.all_gather_object(everyone, [p.numpy() for p in parts])
            return [torch.from_numpy(everyone[src][rank]) for src in range(world)]

        recv = all_to_all(send)                                                     # ids to owners
        back = [torch.from_numpy(my_rows[r.numpy()].astype(np.int32)) for r in recv]  # owner-side gather
        got = all_to_all(back)                                                      # rows back
        gathered = np.empty((rows.size, 64), np.uint16)
        for r in range(world):
            gathered[owner == r] = got[r].numpy().astype(np.uint16)
        mine = po.gather_sum(gathered.reshape(ids.size, 4, 64))                     # slot order, independent of world
        want = po.gather_sum(po.synthetic_table_rows(np.where((rows < 0) | (rows >= total), 0, rows), 64, 9, 0.1))
        assert np.array_equal(mine, want)
        # ---- sharded top-k: per-shard lists, all-gather, merge ------------------------------------------------
        N, k, B = 6000, 50, 4
        clo, chi = pl.shard_range(N, world, rank)
        users = np.random.default_rng(1).standard_normal((B, 32)).astype(np.float32)
        shard = po.synthetic_corpus_rows(np.arange(clo, chi), 32, 3)
        s_loc, i_loc = po.top_k(po.corpus_scores(users, shard), k, row_offset=clo)
        gs = [torch.empty((B, k), dtype=torch.float32) for _ in range(world)]
        gi = [torch.empty((B, k), dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gs, torch.from_numpy(s_loc)); dist.all_gather(gi, torch.from_numpy(i_loc))
        ms, mi = po.merge_top_k([g.numpy() for g in gs], [g.numpy() for g in gi], k)
        ws, wi = po.top_k(po.corpus_scores(users, po.synthetic_corpus_rows(np.arange(N), 32, 3)), k)
        assert np.array_equal(mi, wi) and np.array_equal(ms, ws)
        # the same through the one-word key form the GPU path gathers (one all-gather of 8 bytes per entry)
        gk = [torch.empty((B, k), dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gk, torch.from_numpy(po.topk_keys(s_loc, i_loc).view(np.int64)))
        ks, ki = po.merge_topk_keys([g.numpy().view(np.uint64) for g in gk], k)
        assert np.array_equal(ki, wi) and np.array_equal(ks, ws)
        # ---- data-parallel split: every request served exactly once --------------------------------------------
        served = torch.zeros(11, dtype=torch.int64)
        a, b = pl.split_batch(11, world, rank)
        served[a:b] += 1
        dist.all_reduce(served)
        assert served.tolist() == [1] * 11
        q.put((rank, "ok"))
    except Exception as e:  # surface the failure in the parent
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def test_sharding_plans_world2_gloo():
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res


def test_shard_helpers():
    from x_algorithm_b200 import parallel as pl
    assert [pl.shard_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    o, l = pl.owner_of(np.array([0, 2, 3, 9, 10, -1]), 10, 4)
    assert o.tolist() == [0, 0, 1, 3, 0, 0] and l.tolist() == [0, 2, 0, 0, 0, 0]
    assert [pl.split_batch(7, 3, r) for r in range(3)] == [(0, 3), (3, 5), (5, 7)]
