"""GPU parity at the sizes the benchmarks run: each benchmark configuration at (or near) full shape, through the
default kernel dispatch (no PHX_* switch set), against the CPU oracle on the requests / rows / queries the oracle
finishes in seconds, plus size-independent properties over the rest.  Integer and index work is bit exact; bf16
logits are within 2e-2 relative."""
import math
import os

import numpy as np
import pytest

from oracle import phoenix_oracle as po
from helpers import assert_heads_close, check_topk_against_scores, make_pair, rel_l2, take_requests, to_inputs

pytestmark = pytest.mark.gpu
TOL = 2e-2

# the ranking benchmark's model (bench.py WORKLOAD) with smaller hash regions: the table's size does not change a kernel
CFG1 = dict(emb_size=512, num_layers=8, num_q_heads=8, num_kv_heads=8, key_size=64, widening_factor=4.0,
            history_len=128, num_candidates=512, num_actions=19, num_continuous=1, num_hashes=2, table_size=1 << 16)


@pytest.fixture(scope="module")
def torch():
    import torch
    return torch


@pytest.fixture(autouse=True)
def _no_switches(monkeypatch):
    for k in list(os.environ):
        if k.startswith("PHX_"):
            monkeypatch.delenv(k)


def test_rank_forward_headline_batch_vs_oracle(torch, monkeypatch):
    """B = 256 requests x 512 candidates on the D=512, 8-layer, 8x64-head model, the batch the benchmark times: the
    first, a ragged and the last request against the oracle (logits 2e-2), the kernels the dispatch chose, and hashes /
    summed tokens of those requests bit for bit."""
    import x_algorithm_b200 as px
    from x_algorithm_b200.engine import dispatch_counts
    B = 256
    ocfg, w, rows_fn, eng = make_pair(max_batch=B, **CFG1)
    S, C, H = ocfg.history_len, ocfg.num_candidates, ocfg.num_hashes
    b = po.make_batch(ocfg, B, seed=2, zipf_s=1.1)
    ragged = 100                                           # one request with padded history and candidate tails
    for a in (b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces):
        a[ragged, 57:] = 0
    b.cand_post_ids[ragged, 301:] = 0; b.cand_author_ids[ragged, 301:] = 0
    wt = po.make_blend_weights(1)
    eng.set_blend(px.blend_spec_from_weights(px.ValueModelWeights(w=dict(wt.w)), px.HEAD_NAMES_19, ocfg.num_actions))
    before = dispatch_counts()
    res = eng.rank(to_inputs(b))
    after = dispatch_counts()
    ran = {k: after[k] - before[k] for k in after if after[k] != before[k]}
    # 8 layers: wide CTA-pair tcgen05 GEMMs (4 per layer) and one attention launch per layer on the kernel chosen for
    # head dim 64 with a 128-key history at >= 148 (batch, head) pairs
    assert ran.get("gemm.pair256", 0) == 4 * ocfg.num_layers, ran
    assert sum(v for k, v in ran.items() if k.startswith("gemm.")) == 4 * ocfg.num_layers, ran
    attn = {k: v for k, v in ran.items() if k.startswith("attn.")}
    assert sum(attn.values()) == ocfg.num_layers and len(attn) == 1, ran
    assert list(attn)[0] in ("attn.strip", "attn.resident", "attn.pingpong"), ran     # a resident-history kernel, not the streaming one
    pick = [0, ragged, B - 1]
    sub = take_requests(b, pick)
    taps = {}
    lp, cont, logits = po.rank_forward(ocfg, w, rows_fn, sub, taps)
    valid = sub.cand_post_ids != 0
    stats = assert_heads_close(res.log_probs[pick][valid], res.continuous[pick][valid], logits[valid], cont[valid], TOL,
                               "headline batch")
    print("headline parity:", stats)
    spec = po.blend_spec_from_weights(wt, po.HEAD_NAMES_19, ocfg.num_actions)
    want_s = po.blend_scores(spec, res.log_probs[pick], res.continuous[pick])
    np.testing.assert_allclose(res.scores[pick][valid], want_s[valid], rtol=1e-12, atol=1e-15)
    # the same ragged request alone: a batch of one takes the latency kernels (128-column GEMM tiles, streaming
    # attention), so the bits differ, the answer does not
    alone = eng.rank(to_inputs(take_requests(b, [ragged])))
    assert_heads_close(alone.log_probs[0][valid[1]], alone.continuous[0][valid[1]], logits[1][valid[1]], cont[1][valid[1]], TOL,
                       "one request")
    eng.close()
    # integer / byte stages of the same requests, bit exact (an engine that keeps its per-stage taps)
    monkeypatch.setenv("PHX_DEBUG_TAPS", "1")
    ocfg, w, rows_fn, eng = make_pair(max_batch=B, **CFG1)
    res2 = eng.rank(to_inputs(b))
    T = S + C
    hashes = eng.debug_read("hashes", (B, T, 2 * H), np.int32)[pick]
    want_h = np.concatenate([np.concatenate([taps["hist_post"], taps["hist_author"]], axis=2),
                             np.concatenate([taps["cand_post"], taps["cand_author"]], axis=2)], axis=1)
    np.testing.assert_array_equal(hashes, want_h)
    tokens = eng.debug_read("tokens", (B, T, ocfg.emb_size), np.uint16)[pick]
    np.testing.assert_array_equal(tokens, np.concatenate([taps["hist_tok"], taps["cand_tok"]], axis=1))
    np.testing.assert_array_equal(res2.log_probs, res.log_probs)       # the forward is deterministic
    eng.close()


def test_attention_microbench_shape_vs_oracle(torch):
    """Candidate-isolated attention at the attention benchmark's full shape (batch 64, 16 heads x 128, 1024 history +
    1024 candidates, N(0,1)/sqrt(128) inputs): two batch rows x two heads against the oracle per element, zero rows and
    isolation over the whole output."""
    from x_algorithm_b200.engine import dispatch_counts, ranker_attention
    B, H, dh, S, Cn = 64, 16, 128, 1024, 1024
    T = S + Cn
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = ((torch.randn(B, T, H, dh, device="cuda", generator=g) / math.sqrt(dh)).to(torch.bfloat16) for _ in range(3))
    seg = torch.ones((B, T), dtype=torch.int32, device="cuda")
    seg[:, S:] = -1
    seg[5, 900:S] = 0; seg[5, T - 17:] = 0                   # one row with padded history and candidate tails
    sm = math.sqrt(128.0) / dh
    before = dispatch_counts()
    out, ms = ranker_attention(q, k, v, seg, S, sm)
    after = dispatch_counts()
    assert after["attn.tcgen05"] - before["attn.tcgen05"] == 1
    rows, heads = [5, B - 1], [0, H - 1]
    sl = lambda x: x[rows][:, :, heads].float().cpu().numpy()
    segn = seg[rows].cpu().numpy()
    want = po.masked_attention(sl(q), sl(k), sl(v), po.ranker_mask(segn), sm, -1.0, "soft_sign", po._Rounder("bf16"))
    got = sl(out)
    assert rel_l2(got, want) < TOL
    assert np.abs(got - want).max() < 5 * TOL * float(np.sqrt(np.mean(want ** 2)))
    assert bool((out[5, 900:S] == 0).all()) and bool((out[5, T - 17:] == 0).all())   # padded queries -> zeros
    # isolation at full shape: another candidate's key / value changes nothing but that candidate's own output
    k2, v2 = k.clone(), v.clone()
    k2[:, S + 7] += 1.0; v2[:, S + 7] -= 1.0
    out2, _ = ranker_attention(q, k2, v2, seg, S, sm)
    keep = torch.ones(T, dtype=torch.bool, device="cuda"); keep[S + 7] = False
    assert torch.equal(out[:, keep], out2[:, keep])
    assert not torch.equal(out[:, S + 7], out2[:, S + 7])


def test_gather_sum_benchmark_shape_bit_exact(torch):
    """The gather-sum benchmark's shape on a smaller table: 4 hashes per id, 256-wide bf16 rows, 2^20 Zipf(1.1) ids per
    family.  A strided sample of 32 K ids against the oracle's fixed-order fp32 sum, every id against a second device
    route (row numbers from the hash kernel, rows gathered by the owner-side kernel, summed by the requester-side
    kernel), and equal ids give equal rows."""
    from x_algorithm_b200 import _lib
    lib = _lib.lib
    n, W, Hh = 1 << 20, 256, 4
    ocfg, w, rows_fn, eng = make_pair(emb_size=W, num_hashes=Hh, num_q_heads=W // 64, num_kv_heads=W // 64, key_size=64,
                                      table_size=1 << 20)
    lay = ocfg.hash_layout()
    from x_algorithm_b200.synthetic import zipf_ids
    for fam, hash_fn in ((1, lay.item_hash), (2, lay.author_hash)):
        ids = zipf_ids(n, np.random.Generator(np.random.PCG64(40 + fam)), 1.1)
        ids[:4] = [0, -9, (1 << 40) - 1, 1]
        d_ids = torch.from_numpy(ids).cuda()
        out = torch.empty((n, W), dtype=torch.int16, device="cuda")
        eng.gather_sum_device(fam, d_ids, n, out)
        eng.sync()
        got = out.cpu().numpy().view(np.uint16)
        pick = np.concatenate([np.arange(4), np.arange(5, n, 32)])
        hashed = hash_fn(ids[pick])
        want = po.gather_sum(rows_fn(hashed))
        want[0] = po.gather_sum(rows_fn(np.zeros((1, Hh), np.int32)))[0]           # id 0 reads row 0 for every hash
        np.testing.assert_array_equal(got[pick], want)
        # the second route: hash kernel -> row numbers -> gather kernel -> sum kernel
        rows = torch.empty((n, Hh), dtype=torch.int32, device="cuda")
        eng.hash_ids_device(fam, d_ids, n, rows)
        np.testing.assert_array_equal(rows[pick].cpu().numpy(), hashed)
        table = eng.table_local_ptr()
        gathered = torch.empty((n * Hh, W), dtype=torch.int16, device="cuda")
        out2 = torch.empty_like(out)
        pos = torch.arange(n * Hh, dtype=torch.int32, device="cuda")
        eng.sync()
        torch.cuda.synchronize()
        st = lib.phx_shard_gather_rows(table, ocfg.hash_layout().total_rows, int(rows.data_ptr()), n * Hh, W,
                                       int(gathered.data_ptr()), None)
        assert st == 0, lib.phx_global_error()
        st = lib.phx_shard_sum_rows(int(gathered.data_ptr()), int(pos.data_ptr()), n, Hh, W, int(out2.data_ptr()), None)
        assert st == 0, lib.phx_global_error()
        torch.cuda.synchronize()
        assert torch.equal(out, out2)
        # equal ids -> equal rows (Zipf ids repeat)
        order = np.argsort(ids, kind="stable")
        same = np.flatnonzero(ids[order][1:] == ids[order][:-1])
        assert same.size > 1000
        np.testing.assert_array_equal(got[order[same]], got[order[same + 1]])
    eng.close()


def test_retrieval_benchmark_shape_exact_ids(torch):
    """Top-k = 1000 for 256 queries over a 12.5 M x 128 corpus (one GPU's shard of the 100 M-row retrieval benchmark):
    32 of the queries against fp32 scores of every row computed on the CPU from the corpus bits read back (a sample of
    those bits against the oracle's generator), every query by properties: ordered lists, scores that are the bf16
    rounding of the returned rows' dot products, and the same answer from four row windows merged."""
    from x_algorithm_b200.retrieval import CorpusShard
    from x_algorithm_b200 import _lib
    lib = _lib.lib
    N, dim, k, B, off = 12_500_000, 128, 1000, 256, 25_000_000
    sh = CorpusShard(N, dim, row_offset=off, max_queries=B, max_k=k)
    sh.fill_synthetic(4)
    rng = np.random.default_rng(5)
    u = rng.standard_normal((B, dim)).astype(np.float32)
    u /= np.linalg.norm(u, axis=1, keepdims=True)
    users = torch.from_numpy(u).cuda()
    sc = torch.empty((B, k), dtype=torch.float32, device="cuda"); ids = torch.empty((B, k), dtype=torch.int64, device="cuda")
    sh.topk_device(users, B, k, sc, ids)
    sh.sync()
    got_s, got_i = sc.cpu().numpy(), ids.cpu().numpy()
    # the corpus as the device holds it: a sample of rows against the oracle's generator, then all of it for the scores
    corpus = torch.empty((N, dim), dtype=torch.int16, device="cuda")
    st = lib.phx_corpus_read_device(sh._h, 0, N, int(corpus.data_ptr()))
    assert st == 0
    torch.cuda.synchronize()
    sample = np.concatenate([np.arange(0, N, 9973), [N - 1]])
    np.testing.assert_array_equal(corpus[torch.from_numpy(sample).cuda()].cpu().numpy().view(np.uint16),
                                  po.synthetic_corpus_rows(off + sample, dim, 4))
    nq = 32
    ub = po.bf16_round(u[:nq])                                      # users are rounded to bf16 before the product
    s32 = np.empty((nq, N), np.float32)
    step = 1 << 20
    for r0 in range(0, N, step):
        rows = po.bf16_from_bits(corpus[r0:r0 + step].cpu().numpy().view(np.uint16))
        s32[:, r0:r0 + rows.shape[0]] = ub @ rows.T
    amb = check_topk_against_scores(s32, got_s[:nq], got_i[:nq], k, row_offset=off)
    print("retrieval parity: returned rows within rounding slack of a bf16 boundary:", amb, "of", nq * k)
    del s32
    # every query: order, and scores = bf16(dot) of the returned rows (gathered on the device)
    assert ((got_s[:, 1:] < got_s[:, :-1]) | ((got_s[:, 1:] == got_s[:, :-1]) & (got_i[:, 1:] > got_i[:, :-1]))).all()
    picked = corpus[(ids - off).reshape(-1)].view(torch.bfloat16).float().reshape(B, k, dim)
    dots = torch.einsum("bkd,bd->bk", picked, users.to(torch.bfloat16).float()).cpu().numpy()
    lo, hi = po.bf16_round(dots - np.float32(4e-6)), po.bf16_round(dots + np.float32(4e-6))
    assert ((got_s == lo) | (got_s == hi)).all()
    # four windows, each its own top-k, merged: the same lists
    P = 4
    ws = torch.empty((P, B, k), dtype=torch.float32, device="cuda"); wi = torch.empty((P, B, k), dtype=torch.int64, device="cuda")
    edges = [0, 3_000_001, 6_500_000, 9_999_999, N]
    for p in range(P):
        sh.topk_window_device(users, B, k, edges[p], edges[p + 1], ws[p], wi[p])
    ms_ = torch.empty_like(sc); mi = torch.empty_like(ids)
    sh.merge_device(ws, wi, P, B, k, ms_, mi)
    sh.sync()
    assert torch.equal(mi, ids) and torch.equal(ms_, sc)
    sh.close()
