"""Benchmark of the Phoenix ranking hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step = one ranking forward (hash -> gather-sum -> 8-layer transformer with candidate-isolation
attention -> heads -> weighted blend) over one synthetic batch of 256 requests x 512 candidates
(D=512, 8 heads x 64, FFN 2048, history 128; unified embedding table of 4 x 2^22 rows x 512 bf16).
Prints one JSON line:  value = ranked candidates/s with inputs resident in HBM (CUDA events on the
engine's stream), e2e = the same through the host-buffer C-ABI calls, two requests in flight (each
step's H2D + D2H inside the timed region; `e2e.sync_call` = one blocking call per step), roofline = the GEMM kernel against the measured bf16 peak, cpu_baseline = the NumPy oracle
on the host cores over a bounded sample.  `--impl reference` times the CPU oracle alone.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(emb_size=512, num_layers=8, num_q_heads=8, num_kv_heads=8, key_size=64, widening_factor=4.0,
                history_len=128, num_candidates=512, num_actions=19, num_continuous=1, num_hashes=2,
                table_size=1 << 22)
BATCH = 256
GEMM_DRAM_BYTES_PER_LAUNCH = 714.3e6          # measured (ncu), batch 256, average of the four GEMMs of a layer
GEMM_ALGORITHMIC_BYTES_PER_LAUNCH = 756.6e6   # A + residual + result + weights of the same launches
TABLE_SEED, WEIGHT_SEED, BLEND_SEED, ID_SEED = 7, 0, 1, 2


def flops_per_request(c) -> dict:
    D, F, T = c["emb_size"], int(c["widening_factor"] * c["emb_size"]), c["history_len"] + c["num_candidates"]
    HD = c["num_q_heads"] * c["key_size"]
    QW = (c["num_q_heads"] + 2 * c["num_kv_heads"]) * c["key_size"]
    S, C = c["history_len"], c["num_candidates"]
    # the engine always runs the last layer over the candidate rows only (its history rows are never read again), so
    # at least one layer counts as candidate-only: the FLOPs below are the ones executed, not the dense model's
    L, n_tail = c["num_layers"], max(c.get("num_candidate_only_layers", 0), 1)
    # a candidate-only tail layer projects QKV for every row but runs the out-projection and the FFN over the
    # candidate rows only, and its attention has no history queries
    gemm = L * 2 * T * D * QW + ((L - n_tail) * T + n_tail * C) * (2 * HD * D + 4 * D * F)
    attn = 4 * c["key_size"] * c["num_q_heads"] * ((L - n_tail) * S * S + L * C * (S + 1))
    return dict(gemm=gemm, attn=attn)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16=1400.0, source="fallback")


class ClockSampler(threading.Thread):
    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip().split(",")
                self.samples.append(float(out[0])); self.max_mhz = float(out[1])
                for n, v in zip(names, out[2:]):
                    if v.strip().lower() == "active":
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.05)

    def summary(self):
        return dict(sm_mhz=float(np.median(self.samples)) if self.samples else None, sm_max_mhz=self.max_mhz,
                    reasons=sorted(self.reasons))


def cpu_oracle_rate(n_requests: int, repeats: int = 1, workload=None, batch=None, warmup: int = 0):
    """candidates/s of the NumPy oracle (bf16-emulating path) on `n_requests` requests of the workload (or on the
    requests of `batch`), and the oracle's outputs for them: (rate, seconds, (log_probs, continuous, logits, scores));
    seconds = median of `repeats` passes after `warmup` untimed ones."""
    from oracle import phoenix_oracle as po
    ocfg = po.ModelConfig(**(workload or WORKLOAD), compute="bf16")
    w = po.make_weights(ocfg, WEIGHT_SEED)
    amp = 1.0 / math.sqrt(ocfg.emb_size)
    rows_fn = lambda idx: po.synthetic_table_rows(idx, ocfg.emb_size, TABLE_SEED, amp)
    spec = po.blend_spec_from_weights(po.make_blend_weights(BLEND_SEED), po.HEAD_NAMES_19, ocfg.num_actions)
    b = batch if batch is not None else po.make_batch(ocfg, n_requests, seed=ID_SEED, zipf_s=1.1)
    n_requests = b.cand_post_ids.shape[0]
    times, outs = [], None
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        lp, cont, logits = po.rank_forward(ocfg, w, rows_fn, b)
        sc = po.blend_scores(spec, lp, cont)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
        outs = (lp, cont, logits, sc)
    dt = float(np.median(times))
    return n_requests * ocfg.num_candidates / dt, dt, outs


def run_reference(args, rank: int):
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    n_req = 2
    times = []
    for i in range(args.warmup + args.steps):
        rate, dt, _ = cpu_oracle_rate(n_req)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * float(np.mean(times))
    value = n_req * WORKLOAD["num_candidates"] / (ms / 1e3)
    line = dict(impl="reference", metric="ranked_candidates_per_sec", value=value, unit="candidates/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="bf16", data="synthetic",
                config=dict(workload="phoenix_rank_bf16_D512_L8_H8x64_B256_S128_C512", sample=f"{n_req} requests per step"),
                cpu_baseline=dict(value=value, unit="candidates/s", cores=cores, kind="port",
                                  sample=f"{n_req} requests x 512 candidates per step (NumPy oracle, BLAS threads = all visible cores)"),
                e2e=dict(value=value, unit="candidates/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def sharded_subrecords(args, rank, world, local_rank, steps, which=("gather", "retrieval", "exchange")):
    """N > 1: the three sharded paths, each timed on the device (CUDA events, max over ranks) and checked against the
    unsharded answer on the same GPU.  Returns a dict of sub-records for the JSON line (rank 0's copy is printed).
      sharded_gather     multi-hash gather-sum, 8 x 2^24 x 256 bf16 tables (64 GiB) row-sharded over the ranks, 4 hashes,
                         2^22 Zipf(1.1) ids per step split over the ranks, exchange by the library's communicator
      sharded_retrieval  top-1000 of 256 queries over 100 M x 128 bf16 rows, row-sharded, per-shard scan + all-gather merge
      tables_exchange    the headline ranking step over a row-sharded table, rows fetched by the bulk exchange"""
    import torch
    import torch.distributed as dist
    import x_algorithm_b200 as px
    from x_algorithm_b200 import comm as pc, synthetic
    from x_algorithm_b200.parallel import shard_range
    from x_algorithm_b200.retrieval import CorpusShard
    dev = torch.device("cuda", local_rank)
    peaks = measured_peaks()
    box = [pc.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    cm = pc.Communicator(box[0], rank, world, local_rank)
    out = {}

    per_call = {}

    def timed(fn, iters, warm=2, name=None):
        """ms per call: events on torch's current stream around `iters` calls, max over ranks.  With `name`, the
        duration of every single call (max over ranks) is kept in per_call[name] as well."""
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
        ev[0].record()
        for i in range(iters):
            fn()
            ev[i + 1].record()
        torch.cuda.synchronize()
        t = torch.tensor([ev[0].elapsed_time(ev[iters]) / iters] + [ev[i].elapsed_time(ev[i + 1]) for i in range(iters)],
                         dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if name:
            per_call[name] = [round(float(x), 3) for x in t[1:]]
        return float(t[0])

    def all_true(flag):
        t = torch.tensor([1.0 if flag else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t[0] > 0)

    st = torch.cuda.current_stream().cuda_stream
    # ---- sharded gather-sum ---------------------------------------------------------------------------------------
    try:
        if "gather" not in which:
            raise KeyError("skipped")
        width, hashes, log2_rows, total_ids = 256, 4, 25, 1 << 22
        gcfg = dict(emb_size=width, num_layers=1, num_q_heads=width // 64, num_kv_heads=width // 64, key_size=64,
                    history_len=1, num_candidates=1, max_batch=1, num_hashes=hashes, table_size=1 << log2_rows)
        eng = px.PhoenixEngine(px.PhoenixConfig(table_world=world, table_rank=rank, **gcfg), local_rank)
        eng.table_fill_synthetic(7, 1.0 / math.sqrt(width))
        n = total_ids // world
        sets = [torch.from_numpy(synthetic.zipf_ids(total_ids, np.random.Generator(np.random.PCG64(100 + i)), 1.1)
                                 [rank * n:(rank + 1) * n].copy()).to(dev) for i in range(3)]
        res = torch.empty((n, width), dtype=torch.int16, device=dev)
        cm.gather_setup(eng, n, recv_factor=3.0)
        # a step's ids belong to the four features of the unified table in equal parts (the benchmark's "8 tables" are
        # regions of one row-sharded table here): lookups spread over every shard, as a batch's features do
        fams = [0, 1, 2, 3]
        cnts = [n // 4] * 3 + [n - 3 * (n // 4)]
        it = [0]

        def one():
            cm.gather_sum_multi(eng, fams, cnts, sets[it[0] % 3], res, st)
            it[0] += 1
        ms = timed(one, 10, warm=6, name="gather")   # the warm-up calls also let NCCL finish setting up its send / recv channels
        phases = cm.gather_phase_ms()
        ph_all = [None] * world
        dist.all_gather_object(ph_all, [round(float(x), 3) for x in phases])
        last = it[0] - 1
        whole = px.PhoenixEngine(px.PhoenixConfig(**gcfg), local_rank)
        whole.table_fill_synthetic(7, 1.0 / math.sqrt(width))
        want = torch.empty_like(res)

        def unsharded(ids_t, timed_ms=False):
            at, tot = 0, 0.0
            for f, c in zip(fams, cnts):
                whole.gather_sum_device(f, ids_t[at:at + c], c, want[at:at + c])
                if timed_ms:
                    whole.sync(); tot += whole.last_device_ms()
                at += c
            return tot
        unsharded(sets[0]); whole.sync()
        local_ms = [unsharded(sets[0], True) for _ in range(5)]
        unsharded(sets[last % 3]); whole.sync()
        ok = all_true(torch.equal(res, want))
        whole.close(); eng.close()
        per_id = hashes * width * 2 + width * 2 + 8
        gbs = per_id * total_ids / (ms * 1e-3) / 1e9
        out["sharded_gather"] = dict(
            ms=ms, ids_per_step=total_ids, table_gib=64.0, hashes=hashes, width=width, bytes_per_id=per_id,
            achieved_gbs_aggregate=gbs, frac_of_aggregate_hbm=gbs / (peaks["hbm_gbs"] * world), matches_unsharded=ok,
            one_gpu_share_ms=float(np.median(local_ms)),
            note="one_gpu_share_ms = this rank's ids alone on an unsharded 64 GiB table on the same GPU (no exchange)",
            phase_ms_rank0=dict(zip(["hash_dedup_bucket", "counts_exchange", "row_numbers", "owner_gathers", "copies_tail", "fence", "sum"],
                                    [round(x, 3) for x in phases])),
            ms_per_call=per_call["gather"], phase_ms_last_call_by_rank=ph_all)
    except Exception as e:  # a sub-record must not take the headline line down
        out["sharded_gather"] = dict(error=repr(e))
    # ---- sharded retrieval ----------------------------------------------------------------------------------------
    try:
        if "retrieval" not in which:
            raise KeyError("skipped")
        rows, dim, B, k = 100_000_000, 128, 256, 1000
        lo, hi = shard_range(rows, world, rank)
        sh = CorpusShard(hi - lo, dim, row_offset=lo, max_queries=B, max_k=k, device=local_rank)
        sh.fill_synthetic(4)
        u = np.random.default_rng(5).standard_normal((B, dim)).astype(np.float32)
        u /= np.linalg.norm(u, axis=1, keepdims=True)
        users = torch.from_numpy(u).to(dev)
        sc = torch.empty((B, k), dtype=torch.float32, device=dev); ids = torch.empty((B, k), dtype=torch.int64, device=dev)
        ms = timed(lambda: cm.retrieve_topk(sh, users, B, k, sc, ids, st), 10)
        exact_runs = sh.exact_runs()
        full = CorpusShard(rows, dim, row_offset=0, max_queries=B, max_k=k, device=local_rank)
        full.fill_synthetic(4)
        s2 = torch.empty_like(sc); i2 = torch.empty_like(ids)
        full.topk_device(users, B, k, s2, i2); full.sync()
        one_ms = []
        for _ in range(3):
            full.topk_device(users, B, k, s2, i2); full.sync(); one_ms.append(full.last_device_ms())
        ok = all_true(torch.equal(ids, i2) and torch.equal(sc, s2))
        full.close(); sh.close()
        gbs = rows * dim * 2 / (ms * 1e-3) / 1e9
        out["sharded_retrieval"] = dict(ms=ms, rows=rows, dim=dim, queries=B, k=k, queries_per_s=B / (ms * 1e-3),
                                        corpus_gbs_aggregate=gbs, frac_of_aggregate_hbm=gbs / (peaks["hbm_gbs"] * world),
                                        one_gpu_unsharded_ms=float(np.median(one_ms)), matches_unsharded=ok,
                                        exact_reruns=exact_runs, api="phx_retrieve_topk (blocking; lists + status in one all-gather)")
    except Exception as e:
        out["sharded_retrieval"] = dict(error=repr(e))
    cm.close()
    # ---- ranking over the row-sharded table, rows exchanged in bulk ----------------------------------------------------------
    try:
        if "exchange" not in which:
            raise KeyError("skipped")
        from x_algorithm_b200.parallel import ShardedRanker
        Bq = args.batch
        cfg = px.PhoenixConfig(max_batch=Bq, table_world=world, table_rank=rank, **dict(WORKLOAD, table_size=1 << args.table_log2))
        eng = px.PhoenixEngine(cfg, local_rank)
        eng.load_weights(synthetic.make_weights(cfg, WEIGHT_SEED))
        eng.table_fill_synthetic(TABLE_SEED, 1.0 / math.sqrt(cfg.emb_size))
        bw = synthetic.make_blend_weights(px.HEAD_NAMES_19, BLEND_SEED)
        eng.set_blend(px.blend_spec_from_weights(px.ValueModelWeights(w=bw), px.HEAD_NAMES_19, cfg.num_actions))
        batches = [synthetic.make_batch(cfg, Bq, seed=ID_SEED + 1000 * rank + i, zipf_s=1.1) for i in range(4)]
        db = [[torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in
               (b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces, b.cand_post_ids, b.cand_author_ids)] for b in batches]
        Cn, V, NC = cfg.num_candidates, cfg.num_actions, cfg.num_continuous
        lp = torch.empty((Bq, Cn, V), dtype=torch.float32, device=dev)
        cont = torch.empty((Bq, Cn, NC), dtype=torch.float32, device=dev)
        scs = torch.empty((Bq, Cn), dtype=torch.float64, device=dev)
        ranker = ShardedRanker(eng)

        def step(i):
            ranker.rank_device(Bq, *db[i % 4], lp, cont, scs)
            ranker.prefetch(Bq, *db[(i + 1) % 4])
        for i in range(3):
            step(i)
        eng.sync(); torch.cuda.synchronize(); dist.barrier()
        eng.mark(0)
        for i in range(steps):
            step(i)
        eng.mark(1)
        eng.sync(); torch.cuda.synchronize(); dist.barrier()
        t = torch.tensor([eng.elapsed_ms(0, 1) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # the same batch on an engine with the whole table: bit-identical outputs
        ranker.rank_device(Bq, *db[0], lp, cont, scs); eng.sync()
        got = lp.clone()
        ranker.close(); eng.close()
        whole = px.PhoenixEngine(px.PhoenixConfig(max_batch=Bq, **dict(WORKLOAD, table_size=1 << args.table_log2)), local_rank)
        whole.load_weights(synthetic.make_weights(cfg, WEIGHT_SEED))
        whole.table_fill_synthetic(TABLE_SEED, 1.0 / math.sqrt(cfg.emb_size))
        whole.rank_device(Bq, *db[0], lp, cont, None); whole.sync()
        ok = all_true(torch.equal(got, lp))
        whole.close()
        out["tables_exchange"] = dict(ms_per_step=float(t[0]), value=steps and Bq * Cn * world / (float(t[0]) * 1e-3),
                                      unit="candidates/s", matches_unsharded=ok,
                                      note="headline step with the unified table row-sharded over the ranks; rows of batch i+1 "
                                           "exchanged beside forward i (dedup, bucket, owner gather, copy engines over NVLink)")
    except Exception as e:
        out["tables_exchange"] = dict(error=repr(e))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--table-log2", type=int, default=22, help="log2 buckets per hash region (smaller for profiling captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sharded-only", default="", help="N > 1: skip the headline measurement and run only these sub-records "
                                                       "(comma list of gather, retrieval, exchange); prints them as one JSON line")
    ap.add_argument("--no-sharded-paths", action="store_true",
                    help="N > 1: skip the sharded gather / retrieval / table-exchange sub-records after the headline measurement")
    ap.add_argument("--tables", default="replicated", choices=["sharded", "exchange", "replicated"],
                    help="N > 1: one full table per GPU (it fits: 17 GB); row-sharded over the ranks with per-row peer loads "
                         "over NVLink (sharded); or row-sharded with the bulk row exchange before each forward (exchange: the "
                         "device-timed steps; the host-buffer calls of the e2e leg still use peer loads)")
    ap.add_argument("--candidate-only-layers", type=int, default=0,
                    help="tail layers that update the candidate rows only (the reference's production ranker uses 2; "
                         "the headline workload has none, so a line measured with this flag is not the headline number)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import x_algorithm_b200 as px
    from x_algorithm_b200 import synthetic

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if world > 1 and args.sharded_only:
        sub = sharded_subrecords(args, rank, world, local_rank, args.steps, tuple(args.sharded_only.split(",")))
        if rank == 0:
            print(json.dumps(dict(n_gpus=world, **sub)), flush=True)
        dist.destroy_process_group()
        return

    wl = dict(WORKLOAD)
    wl["table_size"] = 1 << args.table_log2
    if args.candidate_only_layers:
        wl["num_candidate_only_layers"] = args.candidate_only_layers
    B = args.batch
    sharded = world > 1 and args.tables in ("sharded", "exchange")
    exchange = sharded and args.tables == "exchange"
    cfg = px.PhoenixConfig(max_batch=B, table_world=world if sharded else 1, table_rank=rank if sharded else 0, **wl)
    eng = px.PhoenixEngine(cfg, local_rank)
    eng.load_weights(synthetic.make_weights(cfg, WEIGHT_SEED))
    eng.table_fill_synthetic(TABLE_SEED, 1.0 / math.sqrt(cfg.emb_size))
    if sharded:
        from x_algorithm_b200.parallel import attach_table_shards
        attach_table_shards(eng)
    bw = synthetic.make_blend_weights(px.HEAD_NAMES_19, BLEND_SEED)
    eng.set_blend(px.blend_spec_from_weights(px.ValueModelWeights(w=bw), px.HEAD_NAMES_19, cfg.num_actions))

    # synthetic requests: Zipf(1.1) ids over 2^40, a different batch per rank; 4 batches rotated
    n_rot = 4
    batches = [synthetic.make_batch(cfg, B, seed=ID_SEED + 1000 * rank + i, zipf_s=1.1) for i in range(n_rot)]
    dev = torch.device("cuda", local_rank)
    dbatches = [[torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in
                 (b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces, b.cand_post_ids, b.cand_author_ids)]
                for b in batches]
    C, V, NC = cfg.num_candidates, cfg.num_actions, cfg.num_continuous
    lp = torch.empty((B, C, V), dtype=torch.float32, device=dev)
    cont = torch.empty((B, C, NC), dtype=torch.float32, device=dev)
    sc = torch.empty((B, C), dtype=torch.float64, device=dev)
    torch.cuda.synchronize()

    ranker = None
    if exchange:
        from x_algorithm_b200.parallel import ShardedRanker
        ranker = ShardedRanker(eng)

    def step(i):
        # forward of batch i, then (sharded tables) the token gather of batch i+1 on the engine's side stream,
        # which overlaps the forward just enqueued
        if ranker is not None:
            # forward of batch i from the rows exchanged during the previous step, then the exchange of batch i+1
            # beside it
            ranker.rank_device(B, *dbatches[i % n_rot], lp, cont, sc)
            ranker.prefetch(B, *dbatches[(i + 1) % n_rot])
            return
        eng.rank_device(B, *dbatches[i % n_rot], lp, cont, sc)
        if sharded:
            eng.rank_prefetch_device(B, *dbatches[(i + 1) % n_rot])

    for i in range(args.warmup):
        step(i)
    eng.sync()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    eng.mark(0)
    for i in range(args.steps):
        step(i)
    eng.mark(1)
    eng.sync()
    barrier()
    dev_ms = eng.elapsed_ms(0, 1)
    launches = eng.last_launch_count() * args.steps

    # per-kernel-class times of one more step (events around every launch)
    eng.profile_enable(True)
    step(0)
    prof = eng.profile_read()
    eng.profile_enable(False)
    xphase = None
    if ranker is not None:                      # device time of each phase of one exchange (rank 0's view)
        for x in ranker.xchg:
            x.phase_ms = {}
        step(1)
        eng.sync()
        xphase = {}
        for x in ranker.xchg:
            xphase.update(x.phase_ms)
            x.phase_ms = None

    # end to end through the host-buffer call: pinned staging + H2D + forward + D2H inside the timed region
    host_in = [px.RankInputs(b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces, b.cand_post_ids,
                             b.cand_author_ids) for b in batches]
    # two requests in flight (phx_rank_submit / phx_rank_collect): the copies of one overlap the forward of the other;
    # every step still pays its own H2D and D2H inside the timed region.  Result arrays are reused, as a server would.
    outs = [None, None]
    for i in range(2):
        outs[i] = eng.rank(host_in[i % n_rot], None)
    eng.rank_submit(host_in[0], 0); outs[0] = eng.rank_collect(0, outs[0])      # warm the pipelined path
    barrier()
    t0 = time.perf_counter()
    eng.rank_submit(host_in[0], 0)
    for i in range(1, args.steps):
        eng.rank_submit(host_in[i % n_rot], i & 1)
        outs[(i - 1) & 1] = eng.rank_collect((i - 1) & 1, outs[(i - 1) & 1])
    outs[(args.steps - 1) & 1] = eng.rank_collect((args.steps - 1) & 1, outs[(args.steps - 1) & 1])
    out = outs[0]
    e2e_s = time.perf_counter() - t0
    barrier()
    # the same with one blocking call per step (no overlap between steps)
    t0 = time.perf_counter()
    for i in range(args.steps):
        out = eng.rank(host_in[i % n_rot], out)
    e2e_sync_s = time.perf_counter() - t0
    barrier()
    # p50 latency of one request (B=1) and of the throughput batch through the same host-buffer call
    one = px.RankInputs(*[a[:1] for a in (batches[0].hist_post_ids, batches[0].hist_author_ids, batches[0].hist_actions,
                                          batches[0].hist_surfaces, batches[0].cand_post_ids, batches[0].cand_author_ids)])
    lat1, latB = [], []
    out1 = None
    for i in range(1003):      # 3 warm-up calls, then 1000 timed ones
        t1 = time.perf_counter(); out1 = eng.rank(one, out1); lat1.append(time.perf_counter() - t1)
    for i in range(103):
        t1 = time.perf_counter(); eng.rank(host_in[i % n_rot], out); latB.append(time.perf_counter() - t1)
    p50 = dict(request_ms_b1=1e3 * float(np.median(lat1[3:])), request_p99_ms_b1=1e3 * float(np.percentile(lat1[3:], 99)),
               batch_ms=1e3 * float(np.median(latB[3:])), calls_b1=len(lat1) - 3, calls_batch=len(latB) - 3)
    sampler.stop_flag = True
    sampler.join(timeout=2)

    # the engine's answer for batch 0 through the host-buffer call, kept for the parity check below
    check_out = eng.rank(host_in[0], None)
    t = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])

    sub = None
    if world > 1 and not args.no_sharded_paths:
        # The sharded paths are measured by a second set of processes, one per rank, each in a CUDA context of its own
        # (this process gives its device memory back first and then only waits): they hold tables of up to 64 GiB per
        # rank beside an unsharded copy for the check, and a benchmark that starts from a fresh context is the
        # configuration these paths are tested in.  The children form their own process group on the next port.
        if ranker is not None:
            ranker.close(); ranker = None
        eng.close(); eng = None
        del dbatches, lp, cont, sc
        torch.cuda.empty_cache()
        torch.cuda.synchronize()
        dist.barrier()
        # (the launcher's own variables stay behind: with them a child would look for the launcher's rendezvous store
        # on the new port instead of letting its rank 0 open one)
        env = {k_: v_ for k_, v_ in os.environ.items() if not k_.startswith("TORCHELASTIC")}
        env["MASTER_ADDR"] = "127.0.0.1"
        env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + 1)
        cmd = [sys.executable, os.path.abspath(__file__), "--gpus", str(world), "--steps", str(args.steps), "--batch", str(B),
               "--table-log2", str(args.table_log2), "--sharded-only", "gather,retrieval,exchange"]
        try:
            child = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
            lines = [l for l in child.stdout.splitlines() if l.startswith("{")]
            if rank == 0:
                sub = json.loads(lines[-1]) if (child.returncode == 0 and lines) else \
                    dict(sharded_paths=dict(error=f"child exit {child.returncode}: {child.stderr[-400:]}"))
                sub.pop("n_gpus", None)
        except Exception as e:   # the headline line is printed whatever happens to the sub-records
            if rank == 0:
                sub = dict(sharded_paths=dict(error=repr(e)))
        dist.barrier()

    if rank == 0:
        peaks = measured_peaks()
        fl = flops_per_request(wl)
        gemm_ms, gemm_n = prof["gemm"]
        gemm_tflops = fl["gemm"] * B / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        total = args.steps * B * C * world
        h2d = B * (cfg.history_len * 24 + C * 16)
        d2h = B * C * (V * 4 + NC * 4 + 8)
        line = dict(
            metric="ranked_candidates_per_sec", value=total / (dev_ms * 1e-3), unit="candidates/s", n_gpus=world,
            steps=args.steps, warmup=args.warmup, ms_per_step=dev_ms / args.steps, higher_is_better=True, scaling="weak",
            vs_baseline=None, dtype="bf16", data="synthetic",
            config=dict(workload="phoenix_rank_bf16_D512_L8_H8x64_B256_S128_C512", batch_per_gpu=B, history=cfg.history_len,
                        candidates=C, table_rows=cfg.table_rows, parallelism=f"dp{world}",
                        **({"candidate_only_layers": args.candidate_only_layers} if args.candidate_only_layers else {}),
                        tables=("row-sharded over ranks, rows fetched by the bulk exchange before each forward" if exchange else
                                "row-sharded over ranks, remote rows by NVLink peer loads" if sharded else "one full table per GPU"),
                        l2="working set per step (activations 1.7 GB, table 17 GB) exceeds the 126 MB L2; 4 input batches rotated"),
            e2e=dict(value=total / (e2e_ms * 1e-3), unit="candidates/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                     ms_per_step=e2e_ms / args.steps, api="phx_rank_submit / phx_rank_collect, two requests in flight",
                     sync_call=dict(value=B * C * args.steps / e2e_sync_s, ms_per_step=1e3 * e2e_sync_s / args.steps,
                                    api="phx_rank_forward, rank 0")),
            gpu_launches=launches,
            roofline=dict(bound="tensor", kernel="gemm_tcgen05_kernel", achieved=gemm_tflops, peak=peaks["bf16"], unit="TFLOP/s",
                          frac=(gemm_tflops / peaks["bf16"]) if gemm_tflops else None,
                          # dram__bytes_read.sum + dram__bytes_write.sum per launch from an ncu capture of this
                          # command at batch 256 (qkv 620.4, out 459.3, up 784.9, down 992.7 MB: their average), and
                          # the operand + result bytes of the same four launches; both grow with the batch
                          traffic=GEMM_DRAM_BYTES_PER_LAUNCH * (B / 256.0), traffic_unit="bytes/launch",
                          algorithmic_bytes_per_launch=GEMM_ALGORITHMIC_BYTES_PER_LAUNCH * (B / 256.0),
                          peak_source=peaks["source"] + " (sustained bf16)", launches_per_step=gemm_n, ms_per_step=gemm_ms),
            kernel_ms_per_step={k: v[0] for k, v in prof.items()},
            clocks=sampler.summary(),
            p50_latency=p50,
        )
        if xphase is not None:
            line["exchange_phase_ms"] = xphase
        if sub is not None:
            line.update(sub)
        if not args.no_cpu_baseline:
            # The CPU oracle on the first and the last request of batch 0 (outside every timed region): its time is the
            # CPU baseline, its logits are the checker for what the engine returned for the same two requests.
            from oracle import phoenix_oracle as po
            cores = len(os.sched_getaffinity(0))
            pick = [0, B - 1]
            b0 = batches[0]
            sub = po.RankBatch(*[np.ascontiguousarray(getattr(b0, f)[pick]) for f in
                                 ("hist_post_ids", "hist_author_ids", "hist_actions", "hist_surfaces", "cand_post_ids", "cand_author_ids")])
            rate, dt, (o_lp, o_cont, o_logits, o_sc) = cpu_oracle_rate(len(pick), repeats=5, workload=wl, batch=sub, warmup=1)
            line["cpu_baseline"] = dict(value=rate, unit="candidates/s", cores=cores, kind="port",
                                        sample=f"{len(pick)} requests x {C} candidates, median of 5 passes of the NumPy oracle "
                                               f"after 1 warm-up ({dt:.1f} s per pass)")
            g_lp = np.minimum(check_out.log_probs[pick].astype(np.float64), -1e-12)
            g_logits = g_lp - np.log(-np.expm1(g_lp))
            o_logits = o_logits.astype(np.float64)
            dev_c = o_cont.astype(np.float64) - o_cont.astype(np.float64).mean()
            line["parity_check"] = dict(
                requests=pick, against="CPU oracle (bf16-emulating NumPy restatement), same seeded inputs",
                rel_l2_logits=float(np.linalg.norm(g_logits - o_logits) / np.linalg.norm(o_logits)),
                max_abs_logit_err=float(np.abs(g_logits - o_logits).max()), rms_logits=float(np.sqrt(np.mean(o_logits ** 2))),
                rel_l2_continuous_mean_removed=float(np.linalg.norm(check_out.continuous[pick] - o_cont) / np.linalg.norm(dev_c)),
                rel_l2_scores=float(np.linalg.norm(check_out.scores[pick] - o_sc) / np.linalg.norm(o_sc)),
                tolerance=2e-2)
            line["parity_check"]["ok"] = bool(line["parity_check"]["rel_l2_logits"] < 2e-2)
        print(json.dumps(line), flush=True)
    if ranker is not None:
        ranker.close()
    if eng is not None:
        eng.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
