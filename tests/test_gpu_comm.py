"""The library's own communicator (phx_comm_*): sharded retrieval and sharded gather-sum through the C ABI alone, with
no torch.distributed anywhere.  Ranks are child processes, one per GPU; the NCCL unique id travels through a
multiprocessing queue.  A one-rank communicator runs the same code path on a single GPU."""
import math
import multiprocessing as mp
import os
import sys
import traceback

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
N_ROWS, DIM, K, B = 600_000, 128, 200, 24
W_EMB, HASHES, LOG2 = 256, 4, 16
N_IDS = 150_000


def _users():
    rng = np.random.default_rng(5)
    u = rng.standard_normal((B, DIM)).astype(np.float32)
    return u / np.linalg.norm(u, axis=1, keepdims=True)


def _engine(px, world, rank, device):
    cfg = px.PhoenixConfig(emb_size=W_EMB, num_layers=1, num_q_heads=W_EMB // 64, num_kv_heads=W_EMB // 64, key_size=64,
                           history_len=1, num_candidates=1, max_batch=1, num_hashes=HASHES, table_size=1 << LOG2,
                           table_world=world, table_rank=rank)
    eng = px.PhoenixEngine(cfg, device)
    eng.table_fill_synthetic(7, 1.0 / math.sqrt(W_EMB))
    return eng


def _rank_main(rank, world, id_bytes, out_q):
    """One rank: its corpus shard and table shard, one retrieval and two gathers through the communicator; rank 0 also
    computes the unsharded answers on its own GPU and compares."""
    try:
        sys.path.insert(0, ROOT)
        import torch
        import x_algorithm_b200 as px
        from x_algorithm_b200 import comm as pc
        from x_algorithm_b200.parallel import shard_range
        from x_algorithm_b200.retrieval import CorpusShard
        from x_algorithm_b200.synthetic import zipf_ids
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        cm = pc.Communicator(id_bytes, rank, world, rank)
        # retrieval: the same queries on every rank, the corpus split in contiguous row ranges
        lo, hi = shard_range(N_ROWS, world, rank)
        sh = CorpusShard(hi - lo, DIM, row_offset=lo, max_queries=B, max_k=K, device=rank)
        sh.fill_synthetic(4)
        users = torch.from_numpy(_users()).to(dev)
        sc = torch.empty((B, K), dtype=torch.float32, device=dev); ids = torch.empty((B, K), dtype=torch.int64, device=dev)
        cm.retrieve_topk(sh, users, B, K, sc, ids)
        # gather-sum: each rank asks for its own ids, the table is row-sharded
        eng = _engine(px, world, rank, rank)
        cm.gather_setup(eng, N_IDS, recv_factor=4.0)
        gathered = []
        for call in range(2):                                   # twice: the second call reuses every buffer
            my = zipf_ids(N_IDS, np.random.Generator(np.random.PCG64(100 + 10 * call + rank)), 1.1)
            d_ids = torch.from_numpy(my).to(dev)
            out = torch.empty((N_IDS, W_EMB), dtype=torch.int16, device=dev)
            cm.gather_sum(eng, 1 + call, d_ids, N_IDS, out)
            torch.cuda.synchronize()
            gathered.append((my, out, [1 + call], [N_IDS]))
        # a third call with runs of all four features in one exchange (one run empty)
        fams, cnts = [3, 0, 2, 1, 2], [N_IDS // 4, N_IDS // 8, 0, N_IDS // 2, N_IDS - N_IDS // 4 - N_IDS // 8 - N_IDS // 2]
        my = zipf_ids(N_IDS, np.random.Generator(np.random.PCG64(300 + rank)), 1.1)
        out = torch.empty((N_IDS, W_EMB), dtype=torch.int16, device=dev)
        cm.gather_sum_multi(eng, fams, cnts, torch.from_numpy(my).to(dev), out)
        torch.cuda.synchronize()
        gathered.append((my, out, fams, cnts))
        phases = cm.gather_phase_ms()
        ok, msg = True, ""
        # every rank checks its own answers against an unsharded shard / table on its own GPU
        full = CorpusShard(N_ROWS, DIM, row_offset=0, max_queries=B, max_k=K, device=rank)
        full.fill_synthetic(4)
        s2 = torch.empty_like(sc); i2 = torch.empty_like(ids)
        full.topk_device(users, B, K, s2, i2)
        full.sync()
        if not (torch.equal(ids, i2) and torch.equal(sc, s2)):
            ok, msg = False, "sharded retrieval differs from the unsharded scan"
        full.close()
        whole = _engine(px, 1, 0, rank)
        for call, (my, out, fams, cnts) in enumerate(gathered):
            want = torch.empty_like(out)
            d_my, at = torch.from_numpy(my).to(dev), 0
            for f, c in zip(fams, cnts):
                if c:
                    whole.gather_sum_device(f, d_my[at:at + c], c, want[at:at + c])
                at += c
            whole.sync()
            if not torch.equal(out, want):
                ok, msg = False, f"sharded gather-sum (call {call}) differs from the unsharded table"
        whole.close()
        cm.barrier()
        eng.close(); sh.close(); cm.close()
        out_q.put((rank, ok, msg, phases))
    except Exception:
        out_q.put((rank, False, traceback.format_exc(), None))


def _run_world(world):
    sys.path.insert(0, ROOT)
    from x_algorithm_b200 import comm as pc
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    idb = pc.unique_id()
    procs = [ctx.Process(target=_rank_main, args=(r, world, idb, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, ok, msg, phases in sorted(results):
        assert ok, f"rank {rank}: {msg}"
    return results


@pytest.mark.gpu
def test_one_rank_communicator_matches_local_calls():
    _run_world(1)


@pytest.mark.gpu
def test_two_ranks_retrieval_and_gather_match_unsharded():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run_world(2)


def test_communicator_argument_checks():
    """No GPU: the calls refuse bad arguments with PHX_E_ARG before touching CUDA or NCCL."""
    import ctypes as C
    from x_algorithm_b200 import _lib
    lib = _lib.lib
    h = C.c_void_p()
    idb = (C.c_uint8 * 128)()
    assert lib.phx_comm_unique_id(None) == 1
    assert lib.phx_comm_create(None, 0, 1, 0, C.byref(h)) == 1
    assert lib.phx_comm_create(idb, 2, 2, 0, C.byref(h)) == 1            # rank outside the world
    assert lib.phx_comm_create(idb, 0, 0, 0, C.byref(h)) == 1
    assert lib.phx_comm_create(idb, 0, 17, 0, C.byref(h)) == 1           # more ranks than shards the library supports
    assert lib.phx_retrieve_topk(None, None, None, 1, 1, None, None, None) == 1
    assert lib.phx_gather_sum_sharded(None, None, 0, None, 0, None, None) == 1
    assert lib.phx_gather_sum_sharded_multi(None, None, 1, None, None, None, None, None) == 1
    assert lib.phx_gather_sharded_setup(None, None, 10, 2.0) == 1
    assert lib.phx_comm_barrier(None, None) == 1
    assert b"null" in lib.phx_global_error() or b"bad argument" in lib.phx_global_error()
    lib.phx_comm_destroy(None)                                           # a no-op
    st = lib.phx_comm_unique_id(idb)                                     # NCCL present: an id; absent: PHX_E_NCCL with a reason
    assert st in (0, 3)
    if st == 3:
        assert b"NCCL" in lib.phx_global_error()
