"""Micro-benchmarks of the stand-alone operators against their rooflines (one JSON line each).

    python -m x_algorithm_b200.microbench gather  [--ids 4194304] [--log2-rows 25] [--width 256] [--hashes 4]
    torchrun --nproc-per-node N -m x_algorithm_b200.microbench gather [--exchange copy|push|a2a|peer] [--check]
    python -m x_algorithm_b200.microbench topk    [--rows 12500000] [--dim 128] [--queries 256] [--k 1000]
    torchrun --nproc-per-node N -m x_algorithm_b200.microbench retrieve [--rows 100000000] [--check]
    python -m x_algorithm_b200.microbench attention [--batch 64] [--heads 16] [--dh 128] [--hist 1024] [--cands 1024]

gather: the multi-hash gather-sum workload (8 tables x 2^24 rows x 256 bf16 = 64 GiB, realised as the four hash
regions of the unified table x 2^25 rows: the same 2^27 rows x 512 B), 4 hashes per id, Zipf(1.1) ids.
Algorithmic bytes per id = H*W*2 (rows) + W*2 (out) + 8 (id).
topk: exhaustive dot-product top-k over one corpus shard; algorithmic bytes = rows*dim*2.
attention: candidate-isolated attention; algorithmic FLOPs = 4*dh*H*(S^2 + C*(S+1)) per batch element.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import numpy as np


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def _zipf_ids(n, seed, s=1.1):
    from .synthetic import zipf_ids
    return zipf_ids(n, np.random.Generator(np.random.PCG64(seed)), s)


def bench_gather(a):
    import torch
    import x_algorithm_b200 as px
    hbm, _, src = _peaks()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", dev))
    cfg = px.PhoenixConfig(emb_size=a.width, num_layers=1, num_q_heads=a.width // 64, num_kv_heads=a.width // 64,
                           key_size=64, history_len=1, num_candidates=1, max_batch=1, num_hashes=a.hashes,
                           table_size=1 << a.log2_rows, table_world=world, table_rank=rank)
    eng = px.PhoenixEngine(cfg, dev)
    eng.table_fill_synthetic(7, 1.0 / math.sqrt(a.width))
    n = a.ids // world                      # the step's ids are split over the ranks (data parallel), the table is sharded
    sets = [torch.from_numpy(_zipf_ids(a.ids, 100 + i)[rank * n:(rank + 1) * n].copy()).cuda() for i in range(3)]
    out = torch.empty((n, a.width), dtype=torch.int16, device="cuda")
    op = None
    if world > 1:
        from x_algorithm_b200 import parallel
        if a.exchange in ("a2a", "push", "copy"):
            op = parallel.ShardedGatherSum(eng, n, exchange=a.exchange, dedup=not a.no_dedup)
        else:
            parallel.attach_table_shards(eng)
    torch.cuda.synchronize()
    times = []
    for it in range(a.warmup + a.iters):
        fam = it % 4
        if world > 1:
            dist.barrier()
        if op is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            op(fam, sets[it % 3], n, out)
            e1.record()
            torch.cuda.synchronize()
            ms_it = e0.elapsed_time(e1)
        else:
            eng.gather_sum_device(fam, sets[it % 3], n, out)
            eng.sync()
            ms_it = eng.last_device_ms()
        if world > 1:
            t = torch.tensor([ms_it], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_it = float(t[0])
        if it >= a.warmup:
            times.append(ms_it)
    ms = float(np.median(times))
    phases = None
    if op is not None:   # one more call with per-phase device times
        op.phase_ms = {}
        op(0, sets[0], n, out)
        phases = {k: round(v, 3) for k, v in op.phase_ms.items()}
        op.phase_ms = None
    ok = None
    if a.check:   # against an unsharded table on this GPU: bit exact
        full = px.PhoenixEngine(px.PhoenixConfig(emb_size=a.width, num_layers=1, num_q_heads=a.width // 64,
                                                 num_kv_heads=a.width // 64, key_size=64, history_len=1, num_candidates=1,
                                                 max_batch=1, num_hashes=a.hashes, table_size=1 << a.log2_rows), dev)
        full.table_fill_synthetic(7, 1.0 / math.sqrt(a.width))
        want = torch.empty_like(out)
        fam = (a.warmup + a.iters - 1) % 4
        full.gather_sum_device(fam, sets[(a.warmup + a.iters - 1) % 3], n, want)
        full.sync()
        ok = bool(torch.equal(out, want))
        full.close()
        if world > 1:
            t = torch.tensor([1.0 if ok else 0.0], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            ok = bool(t[0] > 0)
    per_id = a.hashes * a.width * 2 + a.width * 2 + 8
    gbs = per_id * n * world / (ms * 1e-3) / 1e9
    if rank == 0:
        print(json.dumps(dict(op="gather_sum", n_gpus=world, exchange=(a.exchange if world > 1 else "local"), ids=n * world,
                              hashes=a.hashes, width=a.width, table_gib=cfg.table_rows * a.width * 2 / 2**30, ms=ms,
                              bytes_per_id=per_id, achieved_gbs=gbs, peak_gbs=hbm * world, frac=gbs / (hbm * world),
                              peak_source=src, matches_unsharded=ok, phase_ms_rank0=phases)))
    if op is not None:
        op.close()
    eng.close()
    if world > 1:
        dist.destroy_process_group()


def bench_topk(a):
    import torch
    from x_algorithm_b200.retrieval import CorpusShard
    hbm, tf, src = _peaks()
    sh = CorpusShard(a.rows, a.dim, row_offset=0, max_queries=a.queries, max_k=a.k)
    sh.fill_synthetic(4)
    if a.int8:                      # the int8 form of the same rows, derived on the device; scores come from it
        sh.quantize_int8()
        sh.set_int8(True)
    rng = np.random.default_rng(5)
    u = rng.standard_normal((a.queries, a.dim)).astype(np.float32)
    u /= np.linalg.norm(u, axis=1, keepdims=True)
    users = torch.from_numpy(u).cuda()
    sc = torch.empty((a.queries, a.k), dtype=torch.float32, device="cuda")
    ids = torch.empty((a.queries, a.k), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    times = []
    for it in range(a.warmup + a.iters):
        sh.topk_device(users, a.queries, a.k, sc, ids)
        sh.sync()
        if it >= a.warmup:
            times.append(sh.last_device_ms())
    ms = float(np.median(times))
    row_bytes = a.dim + 4 if a.int8 else a.dim * 2      # int8 row + its scale, or bf16 row
    gbs = a.rows * row_bytes / (ms * 1e-3) / 1e9
    tfl = 2.0 * a.queries * a.dim * a.rows / (ms * 1e-3) / 1e12
    print(json.dumps(dict(op="corpus_topk_int8" if a.int8 else "corpus_topk", rows=a.rows, dim=a.dim, queries=a.queries, k=a.k, ms=ms, achieved_gbs=gbs,
                          peak_gbs=hbm, frac=gbs / hbm, tflops=tfl, peak_source=src)))
    sh.close()


def bench_retrieve(a):
    """Two-tower retrieval over a row-sharded corpus, one rank per GPU (launch with torchrun): per-shard fused
    top-k -> NCCL all-gather of [B,k] (score, id) -> merge by (score desc, id asc).  --check also scans the whole
    corpus on every rank and demands the identical answer."""
    import torch
    import torch.distributed as dist
    from x_algorithm_b200.retrieval import CorpusShard, Retriever
    from x_algorithm_b200.parallel import shard_range
    hbm, tf, src = _peaks()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lo, hi = shard_range(a.rows, world, rank)
    sh = CorpusShard(hi - lo, a.dim, row_offset=lo, max_queries=a.queries, max_k=a.k, device=local)
    sh.fill_synthetic(4)
    rng = np.random.default_rng(5)
    u = rng.standard_normal((a.queries, a.dim)).astype(np.float32)
    u /= np.linalg.norm(u, axis=1, keepdims=True)
    users = torch.from_numpy(u).cuda()
    ret = Retriever([sh])
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for it in range(a.warmup + a.iters):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev0.record()
        sc, ids = ret.retrieve(users, a.k)
        ev1.record()
        torch.cuda.synchronize()
        if it >= a.warmup:
            times.append(ev0.elapsed_time(ev1))
    t = torch.tensor([float(np.median(times))], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = None
    if a.check:
        full = CorpusShard(a.rows, a.dim, row_offset=0, max_queries=a.queries, max_k=a.k, device=local)
        full.fill_synthetic(4)
        s2 = torch.empty_like(sc); i2 = torch.empty_like(ids)
        full.topk_device(users, a.queries, a.k, s2, i2)
        full.sync()
        ok = bool(torch.equal(ids, i2) and torch.equal(sc, s2))
        full.close()
    if rank == 0:
        ms = float(t[0])
        print(json.dumps(dict(op="retrieve_sharded", n_gpus=world, rows=a.rows, dim=a.dim, queries=a.queries, k=a.k, ms=ms,
                              queries_per_s=a.queries / (ms * 1e-3), corpus_gbs_aggregate=a.rows * a.dim * 2 / (ms * 1e-3) / 1e9,
                              peak_gbs_per_gpu=hbm, frac_of_aggregate_hbm=a.rows * a.dim * 2 / (ms * 1e-3) / 1e9 / (hbm * world),
                              matches_unsharded=ok, peak_source=src)))
    sh.close()
    if world > 1:
        dist.destroy_process_group()


def bench_attention(a):
    import torch
    from x_algorithm_b200.engine import ranker_attention
    _, tf, src = _peaks()
    B, H, dh, S, Cn = a.batch, a.heads, a.dh, a.hist, a.cands
    T = S + Cn
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = ((torch.randn(B, T, H, dh, device="cuda", generator=g) / math.sqrt(dh)).to(torch.bfloat16) for _ in range(3))
    seg = torch.ones((B, T), dtype=torch.int32, device="cuda")
    seg[:, S:] = -1
    times = []
    for it in range(a.warmup + a.iters):
        out, ms = ranker_attention(q, k, v, seg, S, math.sqrt(128.0) / dh)
        if it >= a.warmup:
            times.append(ms)
    ms = float(np.median(times))
    fl = 4.0 * dh * H * (S * S + Cn * (S + 1)) * B
    print(json.dumps(dict(op="ranker_attention", batch=B, heads=H, dh=dh, hist=S, cands=Cn, ms=ms,
                          achieved_tflops=fl / (ms * 1e-3) / 1e12, peak_tflops=tf, frac=fl / (ms * 1e-3) / 1e12 / tf,
                          peak_source=src)))


def bench_gemm(a):
    """The four GEMM shapes of a cfg1 layer at the full M (plain store epilogue), this library's kernel beside
    torch.matmul (cuBLAS) on the same operands: a comparison line, not a path of the engine."""
    import torch
    from x_algorithm_b200.engine import gemm
    M = a.rows_m
    torch.manual_seed(0)
    for name, N, K in (("qkv", 1536, 512), ("out", 512, 512), ("up", 2048, 512), ("down", 512, 2048)):
        x = (torch.randn(M, K, device="cuda") * 0.05).to(torch.bfloat16)
        wt = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)      # [N, K], K-major, as the engine stores weights
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(a.warmup):
            torch.matmul(x, wt.t(), out=out)
        torch.cuda.synchronize()
        lib_ms = []
        for _ in range(a.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch.matmul(x, wt.t(), out=out); e1.record(); torch.cuda.synchronize()
            lib_ms.append(e0.elapsed_time(e1))
        ours_ms = []
        for i in range(a.warmup + a.iters):
            c, ms = gemm(x, wt, None, 0, 0)
            if i >= a.warmup:
                ours_ms.append(ms)
        fl = 2.0 * M * N * K
        t_lib, t_ours = float(np.median(lib_ms)), float(np.median(ours_ms))
        print(json.dumps(dict(op="gemm", shape=name, M=M, N=N, K=K, ms=t_ours, tflops=fl / t_ours / 1e9, cublas_ms=t_lib,
                              cublas_tflops=fl / t_lib / 1e9, ratio_to_cublas=t_lib / t_ours,
                              max_abs_diff=float((c.float() - out.float()).abs().max()))))


def bench_ragged(a):
    """Ragged ranking batches through the blocking host-buffer call, with and without packed rows: the headline benchmark's
    model, --batch requests whose valid history / candidate counts are uniform in [1, S] / [1, C]."""
    import math
    import time
    import x_algorithm_b200 as px
    from x_algorithm_b200 import synthetic
    wl = dict(emb_size=512, num_layers=8, num_q_heads=8, num_kv_heads=8, key_size=64, widening_factor=4.0, history_len=128,
              num_candidates=512, num_actions=19, num_continuous=1, num_hashes=2, table_size=1 << a.log2_rows)
    mcfg = px.PhoenixConfig(max_batch=a.batch, **wl)
    w = synthetic.make_weights(mcfg, 0)
    batch = synthetic.make_batch(mcfg, a.batch, seed=2, ragged=True)
    valid = int((batch.cand_post_ids != 0).sum())
    rows = int((batch.cand_post_ids != 0).sum() + (batch.hist_post_ids != 0).sum())
    inp = px.RankInputs(batch.hist_post_ids, batch.hist_author_ids, batch.hist_actions, batch.hist_surfaces,
                        batch.cand_post_ids, batch.cand_author_ids)
    for pack in (False, True):
        eng = px.PhoenixEngine(px.PhoenixConfig(max_batch=a.batch, pack_ragged=pack, **wl), 0)
        eng.load_weights(w)
        eng.table_fill_synthetic(7, 1.0 / math.sqrt(512))
        out = None
        for i in range(a.warmup + a.iters):
            if i == a.warmup:
                t0 = time.perf_counter()
            out = eng.rank(inp, out)
        dt = (time.perf_counter() - t0) / a.iters
        # the same with two requests in flight (submit / collect)
        outs = [None, None]
        eng.rank_submit(inp, 0)
        for i in range(a.warmup + a.iters):
            if i == a.warmup:
                t1 = time.perf_counter()
            eng.rank_submit(inp, (i + 1) & 1)
            outs[i & 1] = eng.rank_collect(i & 1, outs[i & 1])
        eng.rank_collect((a.warmup + a.iters) & 1)
        dp = (time.perf_counter() - t1) / a.iters
        print(json.dumps(dict(op="rank_ragged", packed=pack, batch=a.batch, valid_candidates=valid, valid_rows=rows,
                              slots=a.batch * 640, ms=dt * 1e3, valid_candidates_per_s=valid / dt,
                              pipelined_ms=dp * 1e3, pipelined_valid_candidates_per_s=valid / dp)))
        eng.close()


def bench_value(a):
    """The value model behind the heads (phx_value_scores_device): --batch requests x --cands candidates, every gate,
    author diversity and class factors on, fuse_heads recomputed (no cached weighted score)."""
    import torch
    from . import value_model as vm
    heads = vm.SCORE_FIELDS[:25]; conts = vm.SCORE_FIELDS[25:]
    rng = np.random.default_rng(3)
    w = {h: float(rng.uniform(0, 5)) for h in heads}
    w.update(report=-80.0, not_interested=-20.0, cont_dwell_time=0.01, video_continuation=0.003, user_video_continuation=0.002)
    wt = vm.ValueModelWeights(w=w, bidirectional_follow_reply_weight_boost=1.0, enable_author_diversity=True,
                              author_diversity_decay=0.6, author_diversity_floor=0.2, oon_rescore_in_network_replies_retweets=True)
    model = vm.value_model_struct(wt, heads, conts)
    B, C = a.batch, a.cands
    g = torch.Generator(device="cuda").manual_seed(1)
    lp = torch.log(torch.rand((B, C, 25), device="cuda", generator=g) * 0.3 + 1e-4)
    cont = torch.rand((B, C, 4), device="cuda", generator=g) * 20
    auth = torch.randint(1, max(2, C // 4), (B, C), device="cuda", generator=g)
    flags = torch.randint(0, 128, (B, C), device="cuda", generator=g).to(torch.uint8)
    lift = torch.full((B, C), -1, dtype=torch.int32, device="cuda"); lift[:, C // 2] = C // 3
    ctx = torch.tensor([[0.75, 0.6, 0.9, 1.2, 0.7]], dtype=torch.float64, device="cuda").repeat(B, 1)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(a.warmup + a.iters):
        if i == a.warmup:
            ev0.record()
        vm.value_scores(model, lp, cont, auth, flags=flags, cold_start_rank=lift, context=ctx)
    ev1.record(); torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / a.iters
    print(json.dumps(dict(op="value_scores", batch=B, candidates=C, ms=ms, candidates_per_s=B * C / (ms * 1e-3),
                          note="includes the two torch.zeros output allocations of the Python wrapper")))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gather", "topk", "attention", "retrieve", "value", "ragged", "gemm"])
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--int8", action="store_true", help="topk: score with the int8 form of the corpus")
    ap.add_argument("--rows-m", type=int, default=163840, help="gemm: rows of the activation matrix")
    ap.add_argument("--no-dedup", action="store_true", help="sharded gather: send every request, not only distinct rows")
    ap.add_argument("--exchange", choices=["copy", "push", "a2a", "peer"], default="copy",
                    help="gather on >1 GPU: owner-side gather + copy-engine transfer into the requester's buffer (copy), "
                         "gather kernel storing into the requester's buffer (push), NCCL all-to-all of the rows (a2a), "
                         "or peer loads inside the requester's kernel (peer)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ids", type=int, default=1 << 22)
    ap.add_argument("--log2-rows", type=int, default=25)
    ap.add_argument("--width", type=int, default=256)
    ap.add_argument("--hashes", type=int, default=4)
    ap.add_argument("--rows", type=int, default=12_500_000)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--queries", type=int, default=256)
    ap.add_argument("--k", type=int, default=1000)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--dh", type=int, default=128)
    ap.add_argument("--hist", type=int, default=1024)
    ap.add_argument("--cands", type=int, default=1024)
    a = ap.parse_args()
    {"gather": bench_gather, "topk": bench_topk, "attention": bench_attention, "retrieve": bench_retrieve,
     "value": bench_value, "ragged": bench_ragged, "gemm": bench_gemm}[a.op](a)


if __name__ == "__main__":
    main()
