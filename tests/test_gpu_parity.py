"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle on the same seeded inputs.
Integer / byte work is bit exact; bf16 floating point is within 2e-2 relative (L2) of the oracle,
the tolerance the workload definition states.  Head outputs are compared as LOGITS (recovered from the
log-probabilities) and as continuous values with their mean removed, each also with a bound on the largest
single error (helpers.assert_heads_close): the log-probabilities and the raw dwell values carry a large
constant part that would hide an error of the part that varies."""
import ctypes as C
import math
import os

import numpy as np
import pytest

from oracle import phoenix_oracle as po
from helpers import assert_heads_close, logits_of, make_pair, rel_l2, to_inputs

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def torch():
    import torch
    return torch


def test_hash_bit_exact_all_families(torch):
    ocfg, w, rows_fn, eng = make_pair()
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "hash_golden.npz"))
    ids = np.concatenate([g["ids"], po.make_batch(ocfg, 64, seed=5, zipf_s=1.1).cand_post_ids.ravel()])
    lay = ocfg.hash_layout()
    want = [lay.user_hash(ids), lay.item_hash(ids), lay.author_hash(ids), lay.ip_hash(ids)]
    d_ids = torch.from_numpy(ids).cuda()
    for fam in range(4):
        out = torch.empty((ids.size, 2), dtype=torch.int32, device="cuda")
        eng.hash_ids_device(fam, d_ids, ids.size, out)
        eng.sync()
        np.testing.assert_array_equal(out.cpu().numpy(), want[fam])
    # the reference function's own outputs for the item family at this bucket count
    np.testing.assert_array_equal(want[1][: g["ids"].size] - lay.offset_item * (want[1][: g["ids"].size] != 0),
                                  g[f"item_{1 << 17}"])
    eng.close()


@pytest.mark.parametrize("emb,hashes", [(128, 2), (256, 4), (512, 2)])
def test_gather_sum_bit_exact(torch, emb, hashes):
    ocfg, w, rows_fn, eng = make_pair(emb_size=emb, num_hashes=hashes, num_q_heads=emb // 32, num_kv_heads=emb // 32,
                                      table_size=1 << 14)
    ids = po.make_batch(ocfg, 32, seed=3, zipf_s=1.1).cand_post_ids.ravel()
    ids[:5] = [0, 1, -7, (1 << 40) - 1, 12345]
    lay = ocfg.hash_layout()
    want = po.gather_sum(rows_fn(lay.item_hash(ids)))
    want[0] = po.gather_sum(rows_fn(np.zeros((1, hashes), np.int32)))[0]   # id 0 -> row 0 for every hash
    d_ids = torch.from_numpy(ids).cuda()
    out = torch.empty((ids.size, emb), dtype=torch.int16, device="cuda")
    eng.gather_sum_device(1, d_ids, ids.size, out)
    eng.sync()
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint16), want)
    eng.close()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 384, 128), (1000, 128, 512), (4096, 1536, 512),
                                   (2048, 512, 2048), (77, 2048, 512)])
@pytest.mark.parametrize("epi", [0, 1, 2])
def test_gemm_tcgen05_vs_fp32(torch, M, N, K, epi):
    from x_algorithm_b200.engine import gemm
    gen = torch.Generator(device="cpu").manual_seed(M + N + K + epi)
    a = (torch.randn(M, K, generator=gen) * 0.5).to(torch.bfloat16).cuda()
    wt = (torch.randn(N, K, generator=gen) * 0.05).to(torch.bfloat16).cuda()
    r = (torch.randn(M, N, generator=gen)).to(torch.bfloat16).cuda() if epi == 1 else None
    ref = a.float() @ wt.float().t()
    ref = ref.to(torch.bfloat16).float()
    if epi == 1:
        ref = ref + r.float()
    elif epi == 2:
        ref = torch.nn.functional.gelu(ref, approximate="tanh")
    ref = ref.to(torch.bfloat16).float()
    for impl in (0, 1, 2):   # tcgen05 with CTA pairs (the default), SIMT cross-check, tcgen05 one CTA per tile
        c, ms = gemm(a, wt, r, epilogue=epi, impl=impl)
        err = rel_l2(c.float().cpu().numpy(), ref.cpu().numpy())
        assert err < 4e-3, (impl, err)
        # elementwise: at most one bf16 ulp apart almost everywhere
        d = (c.float() - ref).abs()
        assert float((d > 0.02 * ref.abs() + 1e-2).float().mean()) < 1e-4, impl


@pytest.mark.parametrize("dh,S,Cn,H", [(32, 32, 8, 4), (64, 128, 64, 2), (128, 96, 40, 2), (64, 200, 56, 3), (128, 300, 200, 1)])
@pytest.mark.parametrize("cap", [(-1.0, 0), (30.0, 1), (30.0, 2)])
@pytest.mark.parametrize("impl", ["tcgen05", "mma", "resident", "strip", "pingpong"])
def test_ranker_attention_vs_oracle(torch, monkeypatch, dh, S, Cn, H, cap, impl):
    """tcgen05/TMEM kernels (head dim 64 / 128; dim 32 falls to mma.sync), the streaming mma.sync kernel, the
    resident-history mma.sync kernel ("strip": head dim 64, <= 128 history keys; other shapes fall through) and the
    resident-history tcgen05 kernel with two softmax warpgroups ("pingpong": the same shapes)."""
    from x_algorithm_b200.engine import ranker_attention
    monkeypatch.setenv("PHX_ATTN", impl)   # "resident" applies to head dim 64 with <= 128 history keys, else tcgen05
    B, T = 3, S + Cn
    rng = np.random.default_rng(dh + S)
    q, k, v = (po.bf16_round(rng.standard_normal((B, T, H, dh)).astype(np.float32)) for _ in range(3))
    pad = np.ones((B, T), bool)
    pad[1, S // 2:S] = False; pad[1, T - 3:] = False        # ragged history and candidates
    pad[2, :S] = False                                       # no history at all: candidates see only themselves
    seg = po.attention_segment_ids(pad, S)
    sm = math.sqrt(128.0) / dh
    method = {0: "soft_sign", 1: "soft_sign", 2: "tanh"}[cap[1]]
    want = po.bf16_round(po.masked_attention(q, k, v, po.ranker_mask(seg), sm, cap[0], method, po._Rounder("bf16")))
    tq, tk, tv = (torch.from_numpy(x).to(torch.bfloat16).cuda() for x in (q, k, v))
    out, ms = ranker_attention(tq, tk, tv, torch.from_numpy(seg).cuda(), S, sm, cap[0], cap[1])
    got = out.float().cpu().numpy()
    assert rel_l2(got, want) < 1e-2
    assert np.abs(got - want).max() < 0.05
    assert (got[seg == 0] == 0).all()                        # padded queries -> zeros
    # candidate isolation: perturbing one candidate's k,v changes only that candidate's output
    k2, v2 = k.copy(), v.copy()
    k2[0, S + 1] += 1.0; v2[0, S + 1] -= 1.0
    out2, _ = ranker_attention(tq, torch.from_numpy(k2).to(torch.bfloat16).cuda(),
                               torch.from_numpy(v2).to(torch.bfloat16).cuda(), torch.from_numpy(seg).cuda(), S, sm,
                               cap[0], cap[1])
    got2 = out2.float().cpu().numpy()
    keep = np.ones(T, bool); keep[S + 1] = False
    np.testing.assert_array_equal(got[0, keep], got2[0, keep])
    assert not np.array_equal(got[0, S + 1], got2[0, S + 1])


@pytest.mark.parametrize("S,Cn,cap", [(128, 512, (-1.0, 0)), (100, 300, (25.0, 2)), (57, 130, (-1.0, 0))])
def test_pingpong_attention_more_items_than_sms(torch, monkeypatch, S, Cn, cap):
    """The persistent two-warpgroup kernel with more (batch, head) items than SMs, so that every CTA walks through
    several items (K / V double buffer, Q ring and the alternation of the warpgroups across item boundaries): four
    batch rows against the oracle, every row against the streaming mma.sync kernel."""
    from x_algorithm_b200.engine import dispatch_counts, ranker_attention
    B, H, dh = 48, 8, 64
    T = S + Cn
    g = torch.Generator(device="cuda").manual_seed(S + Cn)
    q, k, v = (torch.randn(B, T, H, dh, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    seg = torch.ones((B, T), dtype=torch.int32, device="cuda")
    seg[:, S:] = -1
    seg[1, S // 3:S] = 0; seg[1, T - 40:] = 0            # ragged history and candidates
    seg[2, :S] = 0                                       # no history at all
    seg[B - 1, S - 5:S] = 0; seg[B - 1, S + 3] = 0
    sm = math.sqrt(128.0) / dh
    monkeypatch.setenv("PHX_ATTN", "mma")
    want_all, _ = ranker_attention(q, k, v, seg, S, sm, cap[0], cap[1])
    monkeypatch.setenv("PHX_ATTN", "pingpong")
    before = dispatch_counts()
    out, ms = ranker_attention(q, k, v, seg, S, sm, cap[0], cap[1])
    assert dispatch_counts()["attn.pingpong"] - before["attn.pingpong"] == 1
    rows = [0, 1, 2, B - 1]
    sl = lambda x: x[rows].float().cpu().numpy()
    method = "tanh" if cap[1] == 2 else "soft_sign"
    want = po.bf16_round(po.masked_attention(sl(q), sl(k), sl(v), po.ranker_mask(seg[rows].cpu().numpy()), sm, cap[0], method,
                                             po._Rounder("bf16")))
    got = sl(out)
    assert rel_l2(got, want) < 1e-2
    assert np.abs(got - want).max() < 0.05
    a, b = out.float(), want_all.float()
    assert float((a - b).norm() / b.norm()) < 5e-3
    assert bool((out[seg == 0] == 0).all())                               # padded queries -> zeros


@pytest.mark.parametrize("name", ["full", "ragged", "offset", "tanhcap"])
@pytest.mark.parametrize("impl", ["tcgen05", "mma"])
def test_ranker_attention_vs_reference_function_golden(torch, monkeypatch, name, impl):
    """The CUDA kernels against stored outputs of the reference's own plain candidate-isolation attention
    (`attention_reference`, pallas/ranker_attention_fa3.py:1185-1236; tests/golden/attention_golden.npz): bf16 inputs
    (the stored fp32 inputs rounded), so the bar is the bf16 one, 2e-2 relative."""
    import os
    from tests.test_oracle_golden import att_case
    from x_algorithm_b200.engine import ranker_attention
    monkeypatch.setenv("PHX_ATTN", impl)
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz"))
    q, k, v, seg, cand_start, sm, cap, method, want = att_case(g, name)
    tq, tk, tv = (torch.from_numpy(po.bf16_round(x)).to(torch.bfloat16).cuda() for x in (q, k, v))
    out, _ = ranker_attention(tq, tk, tv, torch.from_numpy(seg).cuda(), cand_start, sm, cap,
                              0 if cap <= 0 else (2 if method == "tanh" else 1))
    got = out.float().cpu().numpy()
    assert rel_l2(got, want) < TOL
    assert (got[seg == 0] == 0).all()


def _forward_case(ocfg, w, rows_fn, eng, batch, ragged):
    b = po.make_batch(ocfg, batch, seed=2, ragged=ragged)
    taps = {}
    lp, cont, logits = po.rank_forward(ocfg, w, rows_fn, b, taps)
    wt = po.make_blend_weights(1)
    spec = po.blend_spec_from_weights(wt, po.HEAD_NAMES_19, ocfg.num_actions)
    import x_algorithm_b200 as px
    pw = px.ValueModelWeights(w=dict(wt.w))
    eng.set_blend(px.blend_spec_from_weights(pw, px.HEAD_NAMES_19, ocfg.num_actions))
    res = eng.rank(to_inputs(b))
    return b, taps, lp, cont, logits, spec, res


@pytest.mark.parametrize("ragged", [False, True])
def test_rank_forward_cfg0_vs_oracle(torch, ragged, monkeypatch):
    monkeypatch.setenv("PHX_DEBUG_TAPS", "1")
    ocfg, w, rows_fn, eng = make_pair(max_batch=16)
    B, T, H = 16, ocfg.seq_len, ocfg.num_hashes
    b, taps, lp, cont, logits, spec, res = _forward_case(ocfg, w, rows_fn, eng, B, ragged)
    # integer / byte stages: bit exact
    hashes = eng.debug_read("hashes", (B, T, 2 * H), np.int32)
    want_h = np.concatenate([np.concatenate([taps["hist_post"], taps["hist_author"]], axis=2),
                             np.concatenate([taps["cand_post"], taps["cand_author"]], axis=2)], axis=1)
    np.testing.assert_array_equal(hashes, want_h)
    tokens = eng.debug_read("tokens", (B, T, ocfg.emb_size), np.uint16)
    np.testing.assert_array_equal(tokens, np.concatenate([taps["hist_tok"], taps["cand_tok"]], axis=1))
    # floating point: 2e-2 relative on logits-derived outputs, valid candidates only
    valid = b.cand_post_ids != 0
    assert_heads_close(res.log_probs[valid], res.continuous[valid], logits[valid], cont[valid], TOL, 'forward')
    # against the fp32 path of the oracle as well
    ocfg32 = po.ModelConfig(compute="fp32")
    lp32, cont32, logits32 = po.rank_forward(ocfg32, w, rows_fn, b)
    # (logits only: the bf16 model rounds its dwell prediction to bf16, a step of 1/16 at values near 15, which is
    # already 1e-2 of that head's variation; the fp32 model does not round it)
    assert_heads_close(res.log_probs[valid], None, logits32[valid], None, TOL, "against the fp32 model")
    # blend: exact arithmetic given the engine's own head outputs (f64, same order)
    want_s = po.blend_scores(spec, res.log_probs, res.continuous)
    np.testing.assert_allclose(res.scores[valid], want_s[valid], rtol=1e-12, atol=1e-15)
    assert rel_l2(res.scores[valid], po.blend_scores(spec, lp, cont)[valid]) < 5e-2
    eng.close()


@pytest.mark.parametrize("opts", [dict(qk_norm=True), dict(primer_norm=True), dict(attn_logit_cap=20.0),
                                  dict(attn_logit_cap=20.0, attn_logit_cap_method="tanh", final_logit_cap=10.0),
                                  dict(rotary=False), dict(emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64,
                                                           history_len=48, num_candidates=24, num_layers=3)])
def test_rank_forward_options_vs_oracle(torch, opts):
    ocfg, w, rows_fn, eng = make_pair(max_batch=4, **opts)
    b, taps, lp, cont, logits, spec, res = _forward_case(ocfg, w, rows_fn, eng, 4, True)
    valid = b.cand_post_ids != 0
    assert_heads_close(res.log_probs[valid], res.continuous[valid], logits[valid], cont[valid], TOL, str(opts))
    eng.close()


@pytest.mark.parametrize("opts,attn", [
    (dict(num_candidate_only_layers=1), None),
    (dict(num_candidate_only_layers=2), None),
    (dict(num_candidate_only_layers=1, qk_norm=True), None),
    (dict(num_candidate_only_layers=1, primer_norm=True), None),
    (dict(num_candidate_only_layers=2, emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64, history_len=48,
          num_candidates=24, num_layers=3), "strip"),
    (dict(num_candidate_only_layers=2, emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64, history_len=48,
          num_candidates=300, num_layers=3), "pingpong"),
    (dict(num_candidate_only_layers=2, emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64, history_len=160,
          num_candidates=200, num_layers=3), None),
    (dict(num_candidate_only_layers=3, emb_size=128, num_q_heads=1, num_kv_heads=1, key_size=128, history_len=40,
          num_candidates=24, num_layers=3), None)])
def test_candidate_only_tail_layers_vs_oracle(torch, monkeypatch, opts, attn):
    """The last n layers update the candidate rows only (transformer.py:789-871): history rows stay as the main layers
    left them and every tail layer takes its history keys / values from those rows."""
    if attn:
        monkeypatch.setenv("PHX_ATTN", attn)
    ocfg, w, rows_fn, eng = make_pair(max_batch=5, **opts)
    for batch, ragged in ((5, True), (2, False)):
        b, taps, lp, cont, logits, spec, res = _forward_case(ocfg, w, rows_fn, eng, batch, ragged)
        valid = b.cand_post_ids != 0
        assert_heads_close(res.log_probs[valid], res.continuous[valid], logits[valid], cont[valid], TOL, str(opts))
        # history rows stay as the main layers left them: the first B * S rows of the residual stream (split layout:
        # history block first) equal the output of the model cut after its main layers, not the full model's
        import dataclasses
        S, L, n = ocfg.history_len, ocfg.num_layers, ocfg.num_candidate_only_layers
        hid = eng.debug_read("hidden", (batch * S, ocfg.emb_size), np.uint16).reshape(batch, S, -1)
        hid = po.rms_normalize(po.bf16_from_bits(hid), w["final_norm"], ocfg.rms_eps)
        hv = b.hist_post_ids != 0
        if L > n:
            t_main = {}
            po.rank_forward(dataclasses.replace(ocfg, num_layers=L - n, num_candidate_only_layers=0), w, rows_fn, b, t_main)
            want_hist = t_main["hfin"][:, :S]
        else:   # every layer is a tail layer: the history rows are still the input tokens
            want_hist = po.rms_normalize(taps["x0"][:, :S], w["final_norm"], ocfg.rms_eps)
        t_full = {}
        po.rank_forward(dataclasses.replace(ocfg, num_candidate_only_layers=0), w, rows_fn, b, t_full)
        err_main, err_full = rel_l2(hid[hv], want_hist[hv]), rel_l2(hid[hv], t_full["hfin"][:, :S][hv])
        assert err_main < TOL and err_main < 0.3 * err_full, (opts, err_main, err_full)
    eng.close()


TOL_FP32 = 1e-5   # full-precision path against the fp32 model: the bar set for the full-precision path


@pytest.mark.parametrize("opts", [dict(), dict(qk_norm=True), dict(primer_norm=True),
                                  dict(attn_logit_cap=20.0, attn_logit_cap_method="tanh", final_logit_cap=10.0),
                                  dict(attn_logit_cap=20.0), dict(rotary=False), dict(num_candidate_only_layers=2, num_layers=3),
                                  dict(emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64, history_len=48,
                                       num_candidates=24, num_layers=3)])
def test_rank_forward_fp32_path_vs_fp32_oracle(torch, opts):
    """The CPU-runnable benchmark configuration is an fp32 model: the engine's full-precision path (fp32 activations, SIMT kernels) against the
    oracle's fp32 mode, relative L2 below 1e-5 on the residual stream, log-probabilities and continuous head."""
    ocfg, w, rows_fn, eng = make_pair(max_batch=16, compute="fp32", **opts)
    for batch, ragged in ((16, False), (7, True)):
        b, taps, lp, cont, logits, spec, res = _forward_case(ocfg, w, rows_fn, eng, batch, ragged)
        valid = b.cand_post_ids != 0
        T, S = ocfg.seq_len, ocfg.history_len
        hid = eng.debug_read("hidden", (batch, T, ocfg.emb_size), np.float32)
        hid = po.rms_normalize(hid, w["final_norm"], ocfg.rms_eps)
        tv = np.concatenate([b.hist_post_ids != 0, valid], axis=1)
        assert rel_l2(hid[tv], taps["hfin"][tv]) < TOL_FP32, opts
        assert_heads_close(res.log_probs[valid], res.continuous[valid], logits[valid], cont[valid], TOL_FP32, str(opts))
        want_s = po.blend_scores(spec, res.log_probs, res.continuous)
        np.testing.assert_allclose(res.scores[valid], want_s[valid], rtol=1e-12, atol=1e-15)
        assert rel_l2(res.scores[valid], po.blend_scores(spec, lp, cont)[valid]) < 1e-4
    eng.close()


def test_user_tower_fp32_path_vs_fp32_oracle(torch):
    ocfg, w, rows_fn, eng = make_pair(max_batch=8, compute="fp32", emb_size=128, num_candidates=0, history_len=32)
    b = po.make_batch(po.ModelConfig(history_len=32, num_candidates=1), 8, seed=4, ragged=True)
    want = po.user_tower(ocfg, w, rows_fn, b)
    dev = [torch.from_numpy(x).cuda() for x in (b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces)]
    users = torch.empty((8, 128), dtype=torch.float32, device="cuda")
    eng.user_tower_device(8, *dev, users)
    eng.sync()
    ok = b.hist_post_ids[:, 0] != 0
    assert rel_l2(users.cpu().numpy()[ok], want[ok]) < TOL_FP32
    eng.close()


@pytest.mark.parametrize("opts", [dict(), dict(num_hashes=4, emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64),
                                  dict(num_candidate_only_layers=1)])
def test_rank_forward_from_prehashed_rows_bit_identical(torch, opts):
    """The batch-prep buffers of the reference (rows hashed on the host by its own hash functions,
    recsys_embedding.py:282-331 = the oracle's hash layout) give the same bits as the forward that hashes on the
    device; out-of-table rows read row 0 (emb_table.rs:134-137)."""
    ocfg, w, rows_fn, eng = make_pair(max_batch=6, **opts)
    b = po.make_batch(ocfg, 6, seed=21, ragged=True)
    want = eng.rank(to_inputs(b))
    lay = ocfg.hash_layout()
    hp, ha = lay.item_hash(b.hist_post_ids), lay.author_hash(b.hist_author_ids)
    cp, ca = lay.item_hash(b.cand_post_ids), lay.author_hash(b.cand_author_ids)
    got = eng.rank_hashed(hp, ha, b.hist_actions, b.hist_surfaces, cp, ca)
    np.testing.assert_array_equal(got.log_probs, want.log_probs)
    np.testing.assert_array_equal(got.continuous, want.continuous)
    # device buffers, and a row past the table's end: read as row 0 (the padding row), never out of bounds
    dev = [torch.from_numpy(np.ascontiguousarray(x, np.int32)).cuda() for x in (hp, ha, b.hist_actions, b.hist_surfaces, cp, ca)]
    lp = torch.empty((6, ocfg.num_candidates, ocfg.num_actions), dtype=torch.float32, device="cuda")
    cont = torch.empty((6, ocfg.num_candidates, ocfg.num_continuous), dtype=torch.float32, device="cuda")
    eng.rank_hashed_device(6, *dev, lp, cont)
    eng.sync()
    np.testing.assert_array_equal(lp.cpu().numpy(), want.log_probs)
    ca2 = ca.copy(); ca2[0, 0, 1] = np.iinfo(np.int32).max; ca0 = ca.copy(); ca0[0, 0, 1] = 0
    r_oob = eng.rank_hashed(hp, ha, b.hist_actions, b.hist_surfaces, cp, ca2)
    r_zero = eng.rank_hashed(hp, ha, b.hist_actions, b.hist_surfaces, cp, ca0)
    np.testing.assert_array_equal(r_oob.log_probs, r_zero.log_probs)
    eng.close()


@pytest.mark.parametrize("opts", [dict(), dict(num_candidate_only_layers=1),
                                  dict(num_hashes=4, emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64, history_len=48,
                                       num_candidates=24, num_layers=3)])
def test_projected_tokens_vs_oracle(torch, monkeypatch, opts):
    """The reference's own combine (block_history_reduce / block_candidate_reduce, recsys_model.py:2163-2365): gathered
    rows side by side times a projection matrix.  The gathered operand is a byte copy, so the projected tokens are
    compared before anything else; then the forward."""
    monkeypatch.setenv("PHX_DEBUG_TAPS", "1")
    ocfg, w, rows_fn, eng = make_pair(max_batch=6, token_combine="project", **opts)
    b, taps, lp, cont, logits, spec, res = _forward_case(ocfg, w, rows_fn, eng, 6, True)
    T = ocfg.seq_len
    tokens = po.bf16_from_bits(eng.debug_read("tokens", (6, T, ocfg.emb_size), np.uint16))
    want_tok = po.bf16_from_bits(np.concatenate([taps["hist_tok"], taps["cand_tok"]], axis=1))
    assert rel_l2(tokens, want_tok) < 4e-3          # one bf16 rounding of an fp32 dot product in another summation order
    valid = b.cand_post_ids != 0
    assert_heads_close(res.log_probs[valid], res.continuous[valid], logits[valid], cont[valid], TOL, str(opts))
    # the user tower goes through the same history projection
    want_users = po.user_tower(ocfg, w, rows_fn, b)
    dev = [torch.from_numpy(x).cuda() for x in (b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces)]
    users = torch.empty((6, ocfg.emb_size), dtype=torch.float32, device="cuda")
    eng.user_tower_device(6, *dev, users)
    eng.sync()
    ok = b.hist_post_ids[:, 0] != 0
    assert rel_l2(users.cpu().numpy()[ok], want_users[ok]) < TOL
    eng.close()


@pytest.mark.parametrize("opts,attn", [
    (dict(), None), (dict(num_candidate_only_layers=1), None), (dict(qk_norm=True), None), (dict(token_combine="project"), None),
    (dict(emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64, history_len=48, num_candidates=24, num_layers=3,
          num_candidate_only_layers=2), "strip"),
    (dict(emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64, history_len=160, num_candidates=200, num_layers=2), "mma")])
def test_packed_ragged_batches_match_unpacked(torch, monkeypatch, opts, attn):
    """pack_ragged: the host-buffer call runs a ragged batch over its valid rows only.  Valid candidates get the same
    bits as on the engine that runs every slot (a row's arithmetic does not depend on where the row sits), padded
    candidate slots read zero, and both agree with the oracle.  Also: a request without history, one without
    candidates, a full batch, and a batch that is not front-filled (run over all slots)."""
    if attn:
        monkeypatch.setenv("PHX_ATTN", attn)
    ocfg, w, rows_fn, plain = make_pair(max_batch=6, **opts)
    _, _, _, packed = make_pair(max_batch=6, engine_kw=dict(pack_ragged=True), **opts)
    b = po.make_batch(ocfg, 6, seed=31, ragged=True)
    b.hist_post_ids[1, :] = 0; b.hist_author_ids[1, :] = 0          # no history
    b.cand_post_ids[2, :] = 0; b.cand_author_ids[2, :] = 0          # no candidates
    full = po.make_batch(ocfg, 6, seed=32, ragged=False)
    holes = po.make_batch(ocfg, 6, seed=33, ragged=True)
    holes.cand_post_ids[0, 0] = 0                                   # padding in front of valid slots
    for name, batch in (("ragged", b), ("full", full), ("holes", holes), ("ragged again", b)):
        want = plain.rank(to_inputs(batch))
        got = packed.rank(to_inputs(batch))
        valid = batch.cand_post_ids != 0
        np.testing.assert_array_equal(got.log_probs[valid], want.log_probs[valid], err_msg=name)
        np.testing.assert_array_equal(got.continuous[valid], want.continuous[valid], err_msg=name)
        if name.startswith("ragged"):
            assert (got.log_probs[~valid] == 0).all() and (got.continuous[~valid] == 0).all()
    lp, cont, logits = po.rank_forward(ocfg, w, rows_fn, b)
    valid = b.cand_post_ids != 0
    assert_heads_close(got.log_probs[valid], got.continuous[valid], logits[valid], cont[valid], TOL, "packed rows")
    # two requests in flight through submit / collect: each packs by its own counts
    packed.rank_submit(to_inputs(b), 0)
    packed.rank_submit(to_inputs(full), 1)
    r0, r1 = packed.rank_collect(0), packed.rank_collect(1)
    np.testing.assert_array_equal(r0.log_probs[valid], want.log_probs[valid])
    np.testing.assert_array_equal(r1.log_probs, plain.rank(to_inputs(full)).log_probs)
    assert (r0.log_probs[~valid] == 0).all()
    # device-resident batch with a plan made on the host (phx_plan_ragged + phx_rank_forward_packed_device)
    from x_algorithm_b200.engine import plan_ragged
    ho, co = plan_ragged(b.hist_post_ids, b.cand_post_ids)
    dev = _device_batch(torch, b)
    out = _device_out(torch, packed.cfg, 6)
    packed.rank_packed_device(6, *dev, torch.from_numpy(ho).cuda(), torch.from_numpy(co).cuda(), int(ho[-1]), int(co[-1]), *out[:2])
    packed.sync()
    np.testing.assert_array_equal(out[0].cpu().numpy()[valid], want.log_probs[valid])
    assert (out[0].cpu().numpy()[~valid] == 0).all()
    # the device-pointer entry point of the packing engine runs every slot
    dev = _device_batch(torch, b)
    out = _device_out(torch, packed.cfg, 6)
    packed.rank_device(6, *dev, *out[:2])
    packed.sync()
    np.testing.assert_array_equal(out[0].cpu().numpy()[valid], want.log_probs[valid])
    plain.close(); packed.close()


@pytest.mark.parametrize("opts", [dict(), dict(token_combine="project"), dict(compute="fp32"),
                                  dict(emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64, num_action_types=32)])
def test_action_sets_vs_oracle(torch, monkeypatch, opts):
    """History actions as a set per position (multi_hot_to_embeddings, recsys_model.py:3259-3314): bit masks in
    hist_actions, one [1, D] action vector in signed chunks.  With the row sum the tokens are bit-exact."""
    monkeypatch.setenv("PHX_DEBUG_TAPS", "1")
    ocfg, w, rows_fn, eng = make_pair(max_batch=6, action_multi_hot=True, **opts)
    b, taps, lp, cont, logits, spec, res = _forward_case(ocfg, w, rows_fn, eng, 6, True)
    assert (b.hist_actions == 0).any() and (b.hist_actions > 1).any()
    T = ocfg.seq_len
    tokens = eng.debug_read("tokens", (6, T, ocfg.emb_size), np.uint16)
    want = np.concatenate([taps["hist_tok"], taps["cand_tok"]], axis=1)
    if ocfg.token_combine == "sum":
        np.testing.assert_array_equal(tokens, want)
    else:
        assert rel_l2(po.bf16_from_bits(tokens), po.bf16_from_bits(want)) < 4e-3
    valid = b.cand_post_ids != 0
    tol = TOL_FP32 if ocfg.compute == "fp32" else TOL
    assert_heads_close(res.log_probs[valid], res.continuous[valid], logits[valid], cont[valid], tol, str(opts))
    eng.close()


@pytest.mark.parametrize("opts", [dict(), dict(qk_norm=True), dict(emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64,
                                                                  history_len=48, num_candidates=24, num_layers=3)])
def test_last_layer_runs_candidate_rows_only_bit_identical(torch, monkeypatch, opts):
    """The last layer's history rows are never read again, so the engine runs it over the candidate rows only: the
    same candidate outputs, bit for bit, as with every row computed (PHX_LAST_LAYER=full)."""
    ocfg, w, rows_fn, eng = make_pair(max_batch=5, **opts)
    b = po.make_batch(ocfg, 5, seed=41, ragged=True)
    got = eng.rank(to_inputs(b)); eng.close()
    monkeypatch.setenv("PHX_LAST_LAYER", "full")
    _, _, _, full = make_pair(max_batch=5, **opts)
    want = full.rank(to_inputs(b)); full.close()
    np.testing.assert_array_equal(got.log_probs, want.log_probs)
    np.testing.assert_array_equal(got.continuous, want.continuous)


@pytest.mark.parametrize("opts,attn", [
    (dict(num_q_heads=4, num_kv_heads=2), None), (dict(num_q_heads=4, num_kv_heads=1, qk_norm=True), None),
    (dict(num_q_heads=4, num_kv_heads=2, compute="fp32"), None),
    (dict(emb_size=256, num_q_heads=4, num_kv_heads=2, key_size=64, history_len=48, num_candidates=24, num_layers=3), "strip"),
    (dict(emb_size=256, num_q_heads=4, num_kv_heads=1, key_size=64, history_len=160, num_candidates=72, num_layers=2), None),
    (dict(emb_size=256, num_q_heads=2, num_kv_heads=1, key_size=128, history_len=40, num_candidates=24, num_layers=2), None)])
def test_grouped_query_attention_vs_oracle(torch, monkeypatch, opts, attn):
    """Fewer kv heads than q heads: the merged QKV row keeps the q heads of a kv group together, [q_0..q_{g-1}, k, v]
    (layers.py:728-736), and q head h reads kv head h // g (ranker_attention_v2.py:390)."""
    if attn:
        monkeypatch.setenv("PHX_ATTN", attn)
    ocfg, w, rows_fn, eng = make_pair(max_batch=5, **opts)
    b, taps, lp, cont, logits, spec, res = _forward_case(ocfg, w, rows_fn, eng, 5, True)
    valid = b.cand_post_ids != 0
    tol = TOL_FP32 if ocfg.compute == "fp32" else TOL
    assert_heads_close(res.log_probs[valid], res.continuous[valid], logits[valid], cont[valid], tol, str(opts))
    eng.close()


def test_simt_gemm_path_matches_tcgen05(torch, monkeypatch):
    """The cross-check GEMM and the tcgen05 GEMM give the same forward (accumulation order aside)."""
    ocfg, w, rows_fn, eng = make_pair(max_batch=4)
    b = po.make_batch(ocfg, 4, seed=9)
    r1 = eng.rank(to_inputs(b))
    eng.close()
    monkeypatch.setenv("PHX_GEMM", "simt")
    ocfg, w, rows_fn, eng2 = make_pair(max_batch=4)
    r2 = eng2.rank(to_inputs(b))
    eng2.close()
    assert rel_l2(logits_of(r1.log_probs), logits_of(r2.log_probs)) < 5e-3


def test_row_sharded_table_is_bit_identical(torch, monkeypatch):
    """Two engines each hold half of the unified table and read the other half through a peer mapping (here both on
    one device, attached by pointer; across processes the same path uses CUDA IPC handles).  Hash rows, gathered
    sums and the whole forward are bit-identical to the single-table engine."""
    import x_algorithm_b200 as px
    monkeypatch.setenv("PHX_DEBUG_TAPS", "1")
    ocfg, w, rows_fn, ref = make_pair(max_batch=4)
    amp = 1.0 / math.sqrt(ocfg.emb_size)
    shards = []
    for r in range(2):
        e = px.PhoenixEngine(px.PhoenixConfig(max_batch=4, table_world=2, table_rank=r), 0)
        e.load_weights(w)
        e.table_fill_synthetic(7, amp)
        shards.append(e)
    b = po.make_batch(ocfg, 4, seed=21, ragged=True)
    with pytest.raises(px.PhoenixError) as ei:          # peers not attached yet
        shards[0].rank(to_inputs(b))
    assert ei.value.status == 6 and "not attached" in ei.value.message
    shards[0].table_attach_peer_ptr(1, shards[1].table_local_ptr())
    shards[1].table_attach_peer_ptr(0, shards[0].table_local_ptr())
    want = ref.rank(to_inputs(b))
    want_tok = ref.debug_read("tokens", (4, ocfg.seq_len, ocfg.emb_size), np.uint16)
    for e in shards:
        got = e.rank(to_inputs(b))
        np.testing.assert_array_equal(e.debug_read("tokens", (4, ocfg.seq_len, ocfg.emb_size), np.uint16), want_tok)
        np.testing.assert_array_equal(got.log_probs, want.log_probs)
        np.testing.assert_array_equal(got.continuous, want.continuous)
    ids = po.make_batch(ocfg, 32, seed=3, zipf_s=1.1).cand_post_ids.ravel()
    d_ids = torch.from_numpy(ids).cuda()
    outs = []
    for e in [ref] + shards:
        o = torch.empty((ids.size, ocfg.emb_size), dtype=torch.int16, device="cuda")
        e.gather_sum_device(2, d_ids, ids.size, o)
        e.sync()
        outs.append(o.cpu().numpy())
    np.testing.assert_array_equal(outs[1], outs[0]); np.testing.assert_array_equal(outs[2], outs[0])
    want_rows = po.gather_sum(rows_fn(ocfg.hash_layout().author_hash(ids)))
    np.testing.assert_array_equal(outs[0].view(np.uint16), want_rows)
    for e in shards + [ref]:
        e.close()


def test_token_prefetch_is_transparent(torch):
    """forward(i); prefetch(i+1) pipelining gives bit-identical outputs to plain forwards, also when the prefetched
    batch is not the one that follows (it is discarded)."""
    ocfg, w, rows_fn, eng = make_pair(max_batch=4)
    batches = [po.make_batch(ocfg, 4, seed=30 + i, ragged=True) for i in range(4)]
    want = [eng.rank(to_inputs(b)).log_probs.copy() for b in batches]
    dev = [[torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in
            (b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces, b.cand_post_ids, b.cand_author_ids)]
           for b in batches]
    lp = torch.empty((4, ocfg.num_candidates, ocfg.num_actions), dtype=torch.float32, device="cuda")
    cont = torch.empty((4, ocfg.num_candidates, 1), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    got = []
    eng.rank_prefetch_device(4, *dev[0])
    for i in range(4):
        eng.rank_device(4, *dev[i], lp, cont)
        nxt = (i + 1) % 4 if i != 1 else 3          # after batch 1 prefetch the wrong batch on purpose
        eng.rank_prefetch_device(4, *dev[nxt])
        eng.sync()
        got.append(lp.cpu().numpy().copy())
    for i in range(4):
        np.testing.assert_array_equal(got[i], want[i])
    eng.close()


def test_fused_rmsnorm_matches_separate_kernels(torch, monkeypatch):
    """RMSNorm folded into the GEMMs (gain in the weights, 1/rms applied in the epilogue from row statistics the
    previous GEMM left behind) against the stand-alone norm kernels: same forward up to bf16 rounding noise, and
    both within tolerance of the oracle."""
    ocfg, w, rows_fn, eng = make_pair(max_batch=4, emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64,
                                      history_len=40, num_candidates=24, num_layers=3)
    b = po.make_batch(ocfg, 4, seed=12, ragged=True)
    fused = eng.rank(to_inputs(b)); eng.close()
    monkeypatch.setenv("PHX_NORM", "separate")
    ocfg, w, rows_fn, eng2 = make_pair(max_batch=4, emb_size=256, num_q_heads=4, num_kv_heads=4, key_size=64,
                                       history_len=40, num_candidates=24, num_layers=3)
    sep = eng2.rank(to_inputs(b)); eng2.close()
    lp, cont, logits = po.rank_forward(ocfg, w, rows_fn, b)
    valid = b.cand_post_ids != 0
    assert rel_l2(logits_of(fused.log_probs[valid]), logits_of(sep.log_probs[valid])) < 5e-3
    for r in (fused, sep):
        assert_heads_close(r.log_probs[valid], r.continuous[valid], logits[valid], cont[valid], TOL, "fused / separate norm")


def test_engine_errors_are_statuses(torch):
    import x_algorithm_b200 as px
    with pytest.raises(px.PhoenixError) as ei:
        px.PhoenixEngine(px.PhoenixConfig(key_size=48), 0)
    assert ei.value.status == 1
    eng = px.PhoenixEngine(px.PhoenixConfig(max_batch=2), 0)
    ocfg = po.ModelConfig()
    with pytest.raises(px.PhoenixError) as ei:          # weights not loaded
        eng.rank(to_inputs(po.make_batch(ocfg, 2)))
    assert ei.value.status == 6 and "not loaded" in ei.value.message
    eng.load_weights(po.make_weights(ocfg, 0))
    with pytest.raises(px.PhoenixError) as ei:          # batch beyond capacity
        eng.rank(to_inputs(po.make_batch(ocfg, 3)))
    assert ei.value.status == 5
    # a missing input array is an argument error on every id-path entry point, never a read through a null pointer
    import ctypes as C
    from x_algorithm_b200 import _lib
    b2 = po.make_batch(ocfg, 2)
    arrs = [np.ascontiguousarray(a) for a in (b2.hist_post_ids, b2.hist_author_ids, b2.hist_actions.astype(np.int32),
                                              b2.hist_surfaces.astype(np.int32), b2.cand_post_ids, b2.cand_author_ids)]
    lp = np.empty((2, ocfg.num_candidates, ocfg.num_actions), np.float32)
    cont = np.empty((2, ocfg.num_candidates, ocfg.num_continuous), np.float32)
    o = _lib.RankOut(lp.ctypes.data, cont.ctypes.data, None)
    for missing in range(6):
        ptrs = [a.ctypes.data for a in arrs]
        ptrs[missing] = None
        rb = _lib.RankBatch(2, 0, *ptrs)
        assert _lib.lib.phx_rank_forward(eng._h, C.byref(rb), C.byref(o)) == 1
        assert b"null input array" in _lib.lib.phx_last_error(eng._h)
        assert _lib.lib.phx_rank_forward_device(eng._h, C.byref(rb), C.byref(o)) == 1
        assert _lib.lib.phx_rank_submit(eng._h, C.byref(rb), 0) == 1
    out = eng.rank(to_inputs(po.make_batch(ocfg, 2)))   # the engine stays usable after errors
    assert np.isfinite(out.log_probs).all()
    eng.close()


def test_bounded_device_wait_runs_out_and_engine_stays_usable(torch):
    """Failure detection on the device: a wait on a barrier that nothing signals gives up after the engine's limit (set
    to 1 ms here), the kernel returns, the host reports PHX_E_TIMEOUT once, and the engine keeps working.  Nothing
    faults and nothing hangs: the kernel is one thread polling its own shared-memory barrier."""
    import time
    import x_algorithm_b200 as px
    ocfg, w, rows_fn, eng = make_pair(max_batch=2)
    b = po.make_batch(ocfg, 2, seed=3)
    before = eng.rank(to_inputs(b))
    eng.set_wait_limit_us(1000)
    t0 = time.perf_counter()
    with pytest.raises(px.PhoenixError) as ei:
        eng.wait_selftest()
    dt = time.perf_counter() - t0
    assert ei.value.status == 4 and "bounded device-side wait" in ei.value.message
    assert dt < 1.0, f"the 1 ms limit took {dt:.3f} s to end the wait"
    eng.sync()                                       # the flag was cleared by the call that reported it
    after = eng.rank(to_inputs(b))                   # the same context, the same engine
    np.testing.assert_array_equal(after.log_probs, before.log_probs)
    eng.set_wait_limit_us(0)
    eng.close()


def test_user_tower_and_topk_vs_oracle(torch):
    from x_algorithm_b200.retrieval import CorpusShard, Retriever
    ocfg, w, rows_fn, eng = make_pair(max_batch=8, emb_size=128, num_candidates=0, history_len=32)
    b = po.make_batch(po.ModelConfig(history_len=32, num_candidates=1), 8, seed=4, ragged=True)
    want_users = po.user_tower(ocfg, w, rows_fn, b)
    dev = [torch.from_numpy(x).cuda() for x in (b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces)]
    users = torch.empty((8, 128), dtype=torch.float32, device="cuda")
    eng.user_tower_device(8, *dev, users)
    eng.sync()
    got_users = users.cpu().numpy()
    ok = b.hist_post_ids[:, 0] != 0
    assert rel_l2(got_users[ok], want_users[ok]) < TOL
    # top-k: exact id sets and order (ties -> lower id) for the engine's own user vectors
    N, k = 50_000, 100
    shards = [CorpusShard(N // 2, 128, row_offset=0, max_queries=8, max_k=k),
              CorpusShard(N - N // 2, 128, row_offset=N // 2, max_queries=8, max_k=k)]
    for s in shards:
        s.fill_synthetic(11)
    corpus = po.synthetic_corpus_rows(np.arange(N), 128, 11)
    sc = po.corpus_scores(got_users, corpus)
    want_s, want_i = po.top_k(sc, k)
    got_s, got_i = Retriever(shards).retrieve(users, k)
    np.testing.assert_array_equal(got_i.cpu().numpy(), want_i)
    np.testing.assert_array_equal(got_s.cpu().numpy(), want_s)
    for s in shards:
        s.close()
    eng.close()


@pytest.mark.parametrize("impl,dim", [("tc", 64), ("tc", 128), ("simt", 64), ("simt", 96)])
def test_topk_large_shard_uses_pivot_path(torch, monkeypatch, impl, dim):
    """A shard larger than the survivor capacity goes through the sampled pivot; result still exact.
    Both scan kernels: tcgen05 (dim 64 / 128) and the mma.sync one (any dim % 16 == 0)."""
    from x_algorithm_b200.retrieval import CorpusShard
    if impl == "simt":
        monkeypatch.setenv("PHX_TOPK", "simt")
    N, k, B = 400_000, 64, 20
    sh = CorpusShard(N, dim, row_offset=1000, max_queries=B, max_k=k)
    sh.fill_synthetic(5)
    rng = np.random.default_rng(0)
    u = rng.standard_normal((B, dim)).astype(np.float32)
    u /= np.linalg.norm(u, axis=1, keepdims=True)
    users = torch.from_numpy(u).cuda()
    sc = torch.empty((B, k), dtype=torch.float32, device="cuda"); ids = torch.empty((B, k), dtype=torch.int64, device="cuda")
    sh.topk_device(users, B, k, sc, ids)
    sh.sync()
    corpus = po.synthetic_corpus_rows(np.arange(1000, 1000 + N), dim, 5)
    want_s, want_i = po.top_k(po.corpus_scores(u, corpus), k, row_offset=1000)
    np.testing.assert_array_equal(ids.cpu().numpy(), want_i)
    np.testing.assert_array_equal(sc.cpu().numpy(), want_s)
    sh.close()


@pytest.mark.parametrize("impl,dim,N,windows", [
    ("tc", 128, 60_000, [(0, 60_000), (128, 5_000), (777, 59_999), (30_001, 31_500)]),
    ("tc", 64, 700_000, [(100_003, 650_001), (0, 1_000)]),          # windows larger than the survivor buffer: pivot path
    ("simt", 96, 40_000, [(5, 39_000), (20_000, 21_500)])])
def test_topk_dataset_windows_exact(torch, monkeypatch, impl, dim, N, windows):
    """Top-k restricted to a row window of the shard (the reference's dataset ranges): exact id sets and order against
    the oracle's top-k of the sliced scores, ids offset by the shard's first row and the window's start."""
    from x_algorithm_b200.retrieval import CorpusShard
    if impl == "simt":
        monkeypatch.setenv("PHX_TOPK", "simt")
    B, k, off = 5, 200, 1_000_000
    shard = CorpusShard(N, dim, row_offset=off, max_queries=8, max_k=k)
    shard.fill_synthetic(13)
    corpus = po.synthetic_corpus_rows(np.arange(off, off + N), dim, 13)
    rng = np.random.default_rng(dim)
    users = rng.standard_normal((B, dim)).astype(np.float32)
    users /= np.linalg.norm(users, axis=1, keepdims=True)
    tu = torch.from_numpy(users).cuda()
    sc_all = po.corpus_scores(users, corpus)
    for r0, r1 in windows:
        scores = torch.empty((B, k), dtype=torch.float32, device="cuda"); ids = torch.empty((B, k), dtype=torch.int64, device="cuda")
        shard.topk_window_device(tu, B, k, r0, r1, scores, ids)
        shard.sync()
        want_s, want_i = po.top_k(sc_all[:, r0:r1], k, row_offset=off + r0)
        np.testing.assert_array_equal(ids.cpu().numpy(), want_i)
        # scores are bf16 roundings of fp32 dot products summed in another order: at most one bf16 step apart
        np.testing.assert_allclose(scores.cpu().numpy(), want_s, rtol=2.0 ** -7, atol=0)
    # a window past the shard, an empty one, or one with fewer than k rows is refused
    import x_algorithm_b200 as px
    for bad in ((0, N + 1), (10, 10), (0, k - 1)):
        with pytest.raises(px.PhoenixError):
            shard.topk_window_device(tu, B, k, bad[0], bad[1], scores, ids)
    shard.close()


@pytest.mark.parametrize("impl,dim,N", [("tc", 128, 300_000), ("tc", 64, 700_000), ("simt", 96, 300_000)])
def test_topk_with_row_eligibility_mask(torch, monkeypatch, impl, dim, N):
    """Per-row eligibility (the reference masks a post's score to the bf16 minimum ahead of its top-k,
    recsys_two_tower_model.py:2486-2493): ids equal the oracle's top-k of the scores with masked rows at -inf, for a
    dense and a sparse mask, with windows, and after the mask is lifted."""
    from x_algorithm_b200.retrieval import CorpusShard
    import x_algorithm_b200 as px
    if impl == "simt":
        monkeypatch.setenv("PHX_TOPK", "simt")
    B, k, off = 6, 150, 5_000
    shard = CorpusShard(N, dim, row_offset=off, max_queries=8, max_k=k)
    shard.fill_synthetic(17)
    corpus = po.synthetic_corpus_rows(np.arange(off, off + N), dim, 17)
    rng = np.random.default_rng(N)
    users = rng.standard_normal((B, dim)).astype(np.float32)
    users /= np.linalg.norm(users, axis=1, keepdims=True)
    tu = torch.from_numpy(users).cuda()
    sc_all = po.corpus_scores(users, corpus).astype(np.float32)
    scores = torch.empty((B, k), dtype=torch.float32, device="cuda"); ids = torch.empty((B, k), dtype=torch.int64, device="cuda")

    def check(mask, r0, r1):
        shard.topk_window_device(tu, B, k, r0, r1, scores, ids)
        shard.sync()
        sc = sc_all[:, r0:r1] if mask is None else np.where(mask[None, r0:r1], sc_all[:, r0:r1], -np.inf)
        want_s, want_i = po.top_k(sc, k, row_offset=off + r0)
        np.testing.assert_array_equal(ids.cpu().numpy(), want_i)
        np.testing.assert_allclose(scores.cpu().numpy(), want_s, rtol=2.0 ** -7, atol=0)

    for frac in (0.3, 0.004):
        mask = rng.random(N) < frac
        shard.set_mask(mask)
        check(mask, 0, N)
        check(mask, 1_001, N - 77)
    # fewer eligible rows than k in the window: the reference's top-k runs over the masked scores (masked rows at the
    # bf16 minimum, recsys_two_tower_model.py:2492-2493), so the list ends with the window's first masked rows
    lowest = np.array([0xFF7F0000], np.uint32).view(np.float32)[0]          # finfo(bfloat16).min
    for r0, r1 in ((0, 2_000), (3_001, 3_400)):
        n_el = int(mask[r0:r1].sum())
        assert n_el < k <= r1 - r0
        shard.topk_window_device(tu, B, k, r0, r1, scores, ids)
        shard.sync()
        want_s, want_i = po.top_k(np.where(mask[None, r0:r1], sc_all[:, r0:r1], lowest), k, row_offset=off + r0)
        np.testing.assert_array_equal(ids.cpu().numpy(), want_i)
        got_s = scores.cpu().numpy()
        np.testing.assert_allclose(got_s[:, :n_el], want_s[:, :n_el], rtol=2.0 ** -7, atol=0)
        assert (got_s[:, n_el:] == lowest).all()
    keys = torch.empty((B, k), dtype=torch.int64, device="cuda")           # the same list in key form
    shard.topk_keys_device(tu, B, k, keys)  # (whole shard: enough eligible rows, no padding)
    shard.sync()
    shard.set_mask(None)
    check(None, 0, N)
    shard.close()


@pytest.mark.parametrize("impl,dim", [("tc", 128), ("simt", 96)])
def test_topk_is_exact_when_the_sampled_pivot_misses(torch, monkeypatch, impl, dim):
    """Corpora the sampled pivot cannot serve: every row the same (all scores tie, far more than the survivor buffer
    holds), and a 60,000-row block of copies of one query's direction (that query's top is one long tie).  The sync
    after the call does it again with exact thresholds; ids equal the oracle's top-k, ties to the lower row.  And on
    ordinary rows the exact passes, forced, give what the fast path gives."""
    from x_algorithm_b200.retrieval import CorpusShard, Retriever
    if impl == "simt":
        monkeypatch.setenv("PHX_TOPK", "simt")
    N, k, B, off = 400_000, 100, 6, 7_000
    rng = np.random.default_rng(dim)
    u = rng.standard_normal((B, dim)).astype(np.float32)
    u /= np.linalg.norm(u, axis=1, keepdims=True)
    users = torch.from_numpy(u).cuda()
    sc = torch.empty((B, k), dtype=torch.float32, device="cuda"); ids = torch.empty((B, k), dtype=torch.int64, device="cuda")
    sh = CorpusShard(N, dim, row_offset=off, max_queries=8, max_k=k)

    def run_and_check(corpus_bits, want_reruns):
        sh.upload(0, corpus_bits)
        before = sh.exact_runs()
        sh.topk_device(users, B, k, sc, ids)
        reran = sh.finish()
        assert reran == (want_reruns > 0) and sh.exact_runs() - before == want_reruns
        want_s, want_i = po.top_k(po.corpus_scores(u, corpus_bits), k, row_offset=off)
        np.testing.assert_array_equal(ids.cpu().numpy(), want_i)
        np.testing.assert_allclose(sc.cpu().numpy(), want_s, rtol=2.0 ** -7, atol=0)

    base = po.synthetic_corpus_rows(np.arange(off, off + N), dim, 29)
    same = np.repeat(base[:1], N, axis=0)
    run_and_check(same, 1)                                   # the k lowest rows, for every query
    np.testing.assert_array_equal(ids.cpu().numpy(), np.tile(np.arange(off, off + k), (B, 1)))
    block = base.copy()
    block[300_000:360_000] = po.bf16_bits(u[0])[None, :]     # 60,000 copies of query 0's direction
    run_and_check(block, 1)
    assert (ids[0].cpu().numpy() == np.arange(off + 300_000, off + 300_000 + k)).all()
    run_and_check(base, 0)                                   # ordinary rows: the fast path serves them
    fast_i, fast_s = ids.clone(), sc.clone()
    sh.set_exact(True)
    sh.topk_device(users, B, k, sc, ids)
    sh.sync()
    sh.set_exact(False)
    assert torch.equal(ids, fast_i) and torch.equal(sc, fast_s)
    # through the retriever: the merged answer is exact too, the re-run replaces the shard's list before the merge
    sh.upload(0, block)
    got_s, got_i = Retriever([sh]).retrieve(users, k)
    want_s, want_i = po.top_k(po.corpus_scores(u, block), k, row_offset=off)
    np.testing.assert_array_equal(got_i.cpu().numpy(), want_i)
    sh.close()


def test_retriever_orders_its_work_on_the_callers_stream(torch):
    """Retriever.retrieve enqueues per-shard top-k (as 64-bit keys), the merge and anything the caller adds on torch's
    current stream, default stream included, with no host synchronisation in between: reading the result right away
    must give the oracle's answer, on shards large enough for a race to show."""
    from x_algorithm_b200.retrieval import CorpusShard, Retriever
    N, dim, k, B = 600_000, 64, 100, 8
    shards = [CorpusShard(N // 2, dim, row_offset=0, max_queries=B, max_k=k), CorpusShard(N - N // 2, dim, row_offset=N // 2, max_queries=B, max_k=k)]
    for sh in shards:
        sh.fill_synthetic(23)
    rng = np.random.default_rng(7)
    u = rng.standard_normal((B, dim)).astype(np.float32)
    u /= np.linalg.norm(u, axis=1, keepdims=True)
    users = torch.from_numpy(u).cuda()
    want_s, want_i = po.top_k(po.corpus_scores(u, po.synthetic_corpus_rows(np.arange(N), dim, 23)), k)
    ret = Retriever(shards)
    for stream in (torch.cuda.current_stream(), torch.cuda.Stream()):
        with torch.cuda.stream(stream):
            sc, ids = ret.retrieve(users, k)
            doubled = sc * 2           # the caller's own work behind the merge, same stream
            got_i, got_d = ids.cpu().numpy(), doubled.cpu().numpy()
        np.testing.assert_array_equal(got_i, want_i)
        np.testing.assert_allclose(got_d, 2 * want_s, rtol=2.0 ** -7, atol=0)
    # the per-shard list in key form decodes to the oracle's list of that shard, and the oracle's merge of the two
    # shards' device-made keys is the global answer
    dev_keys = []
    for p, sh in enumerate(shards):
        keys = torch.empty((B, k), dtype=torch.int64, device="cuda")
        sh.set_stream(None)
        sh.topk_keys_device(users, B, k, keys)
        sh.sync()
        dev_keys.append(keys.cpu().numpy().view(np.uint64))
        lo = p * (N // 2)
        rows = po.synthetic_corpus_rows(np.arange(lo, lo + sh.rows), dim, 23)
        ws, wi = po.top_k(po.corpus_scores(u, rows), k, row_offset=lo)
        ds, di = po.merge_topk_keys([dev_keys[-1]], k)
        np.testing.assert_array_equal(di, wi)
        np.testing.assert_allclose(ds, ws, rtol=2.0 ** -7, atol=0)
    np.testing.assert_array_equal(po.merge_topk_keys(dev_keys, k)[1], want_i)
    for sh in shards:
        sh.close()


def test_sharded_gather_exchange_kernels_bit_identical(torch):
    """The device-side steps of the all-to-all exchange (bucket by owner, owner-side gather, fixed-order sum), with
    the two collectives emulated by slicing: two "ranks" on one device, each holding half of the table.  The result
    is bit-identical to the gather-sum over the unsharded table."""
    import x_algorithm_b200 as px
    from x_algorithm_b200 import _lib
    from x_algorithm_b200.engine import _ptr
    from x_algorithm_b200.parallel import rows_per_shard
    lib = _lib.lib
    W, n, width, H = 2, 5000, 256, 4
    mk = lambda **kw: px.PhoenixConfig(emb_size=width, num_layers=1, num_q_heads=4, num_kv_heads=4, key_size=64, history_len=1,
                                       num_candidates=1, max_batch=1, num_hashes=H, table_size=1 << 12, **kw)
    full = px.PhoenixEngine(mk(), 0)
    full.table_fill_synthetic(7, 0.0625)
    shards = [px.PhoenixEngine(mk(table_world=W, table_rank=r), 0) for r in range(W)]
    for e in shards:
        e.table_fill_synthetic(7, 0.0625)
    rps = rows_per_shard(full.cfg.table_rows, W)
    rng = np.random.default_rng(3)
    ids = [torch.from_numpy(rng.integers(-2**40, 2**40, n).astype(np.int64)).cuda() for _ in range(W)]
    ids[0][:3] = 0                                              # id 0 -> row 0 for every hash
    i32 = dict(dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rows, send, pos, counts = [], [], [], []
    for r in range(W):
        rw = torch.empty(n * H, **i32)
        shards[r].hash_ids_device(1, ids[r], n, rw); shards[r].sync()
        sr, ps, ct, cur = torch.empty(n * H, **i32), torch.empty(n * H, **i32), torch.empty(W, **i32), torch.empty(W, **i32)
        assert lib.phx_shard_bucket(_ptr(rw), n * H, rps, W, _ptr(ct), _ptr(cur), _ptr(sr), _ptr(ps), st) == 0
        torch.cuda.synchronize()
        rows.append(rw); send.append(sr); pos.append(ps); counts.append(ct.tolist())
        assert sum(counts[r]) == n * H
        owner = (rw.cpu().numpy() // rps)
        assert counts[r] == [int((owner == o).sum()) for o in range(W)]
        # every request landed in its owner's bucket with the right local row
        base = np.concatenate([[0], np.cumsum(counts[r])])
        p_np, s_np, r_np = ps.cpu().numpy(), sr.cpu().numpy(), rw.cpu().numpy()
        assert sorted(p_np.tolist()) == list(range(n * H))
        assert ((p_np >= base[owner]) & (p_np < base[owner + 1])).all()
        np.testing.assert_array_equal(s_np[p_np], r_np - owner * rps)
    # "all-to-all" of the row numbers, owner-side gather, "all-to-all" of the rows
    back = [torch.empty((n * H, width), dtype=torch.int16, device="cuda") for _ in range(W)]
    for o in range(W):
        parts = []
        for r in range(W):
            b0 = sum(counts[r][:o])
            parts.append(send[r][b0:b0 + counts[r][o]])
        req = torch.cat(parts)
        got = torch.empty((req.numel(), width), dtype=torch.int16, device="cuda")
        assert lib.phx_shard_gather_rows(shards[o].table_local_ptr(), rps, _ptr(req), req.numel(), width, _ptr(got), st) == 0
        off = 0
        for r in range(W):
            b0 = sum(counts[r][:o])
            back[r][b0:b0 + counts[r][o]] = got[off:off + counts[r][o]]
            off += counts[r][o]
    for r in range(W):
        out = torch.empty((n, width), dtype=torch.int16, device="cuda")
        assert lib.phx_shard_sum_rows(_ptr(back[r]), _ptr(pos[r]), n, H, width, _ptr(out), st) == 0
        want = torch.empty_like(out)
        full.gather_sum_device(1, ids[r], n, want); full.sync()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    # duplicate requests folded first: distinct rows -> bucket -> positions expanded back to every request
    r = 0
    dup_ids = ids[r].clone(); dup_ids[n // 2:] = dup_ids[:n - n // 2]          # every id (at least) twice
    rw = torch.empty(n * H, **i32)
    shards[r].hash_ids_device(1, dup_ids, n, rw); shards[r].sync()
    slots = 1 << 16
    table = torch.empty(slots, dtype=torch.int64, device="cuda")
    slot, urows, upos, ps2 = (torch.empty(n * H, **i32) for _ in range(4))
    nu = torch.empty(1, **i32)
    assert lib.phx_shard_dedup(_ptr(rw), n * H, _ptr(table), slots, _ptr(slot), _ptr(urows), _ptr(nu), st) == 0
    nuq = int(nu.item())
    assert nuq == len(np.unique(rw.cpu().numpy())) and nuq <= n * H // 2 + H * 3
    np.testing.assert_array_equal(np.sort(urows[:nuq].cpu().numpy()), np.unique(rw.cpu().numpy()))
    sr, ct, cur = torch.empty(n * H, **i32), torch.empty(W, **i32), torch.empty(W, **i32)
    assert lib.phx_shard_bucket(_ptr(urows), nuq, rps, W, _ptr(ct), _ptr(cur), _ptr(sr), _ptr(upos), st) == 0
    assert lib.phx_shard_dedup_expand(_ptr(slot), _ptr(table), _ptr(upos), n * H, _ptr(ps2), st) == 0
    torch.cuda.synchronize()
    cts = ct.tolist()
    landing = torch.empty((nuq, width), dtype=torch.int16, device="cuda")
    for o in range(W):
        b0 = sum(cts[:o])
        assert lib.phx_shard_gather_rows(shards[o].table_local_ptr(), rps, _ptr(sr) + 4 * b0, cts[o], width,
                                         _ptr(landing) + 2 * width * b0, st) == 0
    out = torch.empty((n, width), dtype=torch.int16, device="cuda")
    assert lib.phx_shard_sum_rows(_ptr(landing), _ptr(ps2), n, H, width, _ptr(out), st) == 0
    want = torch.empty_like(out)
    full.gather_sum_device(1, dup_ids, n, want); full.sync()
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert lib.phx_shard_dedup(_ptr(rw), n * H, _ptr(table), 1000, _ptr(slot), _ptr(urows), _ptr(nu), st) == 1   # not a power of two
    assert lib.phx_shard_bucket(0, 1, rps, W, 0, 0, 0, 0, st) == 1        # PHX_E_ARG on null pointers
    for e in shards + [full]:
        e.close()


def test_graph_replay_matches_eager(torch, monkeypatch):
    """A host-buffer call that repeats the previous call's batch size is captured into a CUDA graph and replayed:
    outputs identical to the eager launches, also after the inputs' contents change and after the blend is reset."""
    ocfg, w, rows_fn, eng = make_pair(max_batch=8)
    b1 = po.make_batch(ocfg, 8, seed=31, ragged=True)
    b2 = po.make_batch(ocfg, 8, seed=32, ragged=False)
    monkeypatch.setenv("PHX_GRAPH", "0")
    ocfg, w, rows_fn, eager = make_pair(max_batch=8)
    want1, want2 = eager.rank(to_inputs(b1)), eager.rank(to_inputs(b2))
    eager.close()
    monkeypatch.delenv("PHX_GRAPH")
    got = [eng.rank(to_inputs(b)) for b in (b1, b1, b1, b2, b2, b1)]      # eager, capture, replay, replay with new data ...
    for g, wnt in zip(got, (want1, want1, want1, want2, want2, want1)):
        np.testing.assert_array_equal(g.log_probs, wnt.log_probs)
        np.testing.assert_array_equal(g.continuous, wnt.continuous)
        np.testing.assert_array_equal(g.scores, wnt.scores)
    small = po.make_batch(ocfg, 3, seed=33, ragged=True)                  # another batch size: new key, eager again
    ocfg2, w2, rows_fn2, ref = make_pair(max_batch=8)
    np.testing.assert_array_equal(eng.rank(to_inputs(small)).log_probs, ref.rank(to_inputs(small)).log_probs)
    ref.close()
    eng.close()


def test_pipelined_submit_collect_matches_blocking_call(torch):
    """Two requests in flight through phx_rank_submit / phx_rank_collect give the results of the blocking call,
    whatever the order of collection; a slot cannot be resubmitted before it is collected."""
    import x_algorithm_b200 as px
    ocfg, w, rows_fn, eng = make_pair(max_batch=8)
    bs = [po.make_batch(ocfg, n, seed=40 + i, ragged=bool(i & 1)) for i, n in enumerate((8, 5, 8, 1))]
    want = [eng.rank(to_inputs(b)) for b in bs]
    eng.rank_submit(to_inputs(bs[0]), 0)
    eng.rank_submit(to_inputs(bs[1]), 1)
    with pytest.raises(px.PhoenixError) as ei:
        eng.rank_submit(to_inputs(bs[2]), 1)
    assert ei.value.status == 6
    got0 = eng.rank_collect(0)
    eng.rank_submit(to_inputs(bs[2]), 0)
    got1 = eng.rank_collect(1)
    eng.rank_submit(to_inputs(bs[3]), 1)
    got3 = eng.rank_collect(1)
    got2 = eng.rank_collect(0)
    for g, wnt in zip((got0, got1, got2, got3), want):
        np.testing.assert_array_equal(g.log_probs, wnt.log_probs)
        np.testing.assert_array_equal(g.continuous, wnt.continuous)
    with pytest.raises(px.PhoenixError):
        eng.rank_collect(0)
    eng.close()


def _device_batch(torch, b):
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dt)).cuda()
    return (t(b.hist_post_ids, np.int64), t(b.hist_author_ids, np.int64), t(b.hist_actions, np.int32),
            t(b.hist_surfaces, np.int32), t(b.cand_post_ids, np.int64), t(b.cand_author_ids, np.int64))


def _device_out(torch, cfg, B):
    return (torch.empty((B, cfg.num_candidates, cfg.num_actions), dtype=torch.float32, device="cuda"),
            torch.empty((B, cfg.num_candidates, cfg.num_continuous), dtype=torch.float32, device="cuda"))


def test_forward_from_exchanged_rows_bit_identical(torch):
    """phx_rank_rows_device + phx_rank_forward_rows_device (the two halves of a forward around a row exchange):
    the rows it names are those of the oracle's hashes, and the forward over a shuffled, de-duplicated landing
    buffer equals the forward over the table bit for bit (ragged batch: padded slots name row 0)."""
    from x_algorithm_b200 import _lib
    from x_algorithm_b200.engine import _ptr
    ocfg, w, rows_fn, eng = make_pair(max_batch=8)
    cfg, B = eng.cfg, 7
    b = po.make_batch(ocfg, B, seed=51, ragged=True)
    dev = _device_batch(torch, b)
    want = _device_out(torch, cfg, B)
    eng.rank_device(B, *dev, *want); eng.sync()
    T, H2 = cfg.history_len + cfg.num_candidates, 2 * cfg.num_hashes
    rows = torch.empty(B * T * H2, dtype=torch.int32, device="cuda")
    eng.rank_rows_device(B, *dev, rows); eng.sync()
    r = rows.cpu().numpy().reshape(B, T, H2)
    post = np.concatenate([b.hist_post_ids, b.cand_post_ids], 1)
    auth = np.concatenate([b.hist_author_ids, b.cand_author_ids], 1)
    lay = ocfg.hash_layout()
    np.testing.assert_array_equal(r[..., :cfg.num_hashes], lay.item_hash(post))
    np.testing.assert_array_equal(r[..., cfg.num_hashes:], lay.author_hash(auth))
    urows, inv = torch.unique(rows, return_inverse=True)
    perm = torch.randperm(urows.numel(), device="cuda", generator=torch.Generator("cuda").manual_seed(5))
    where = torch.empty_like(perm); where[perm] = torch.arange(perm.numel(), device="cuda")
    landing = torch.empty((urows.numel(), cfg.emb_size), dtype=torch.bfloat16, device="cuda")
    shuffled = urows[perm].to(torch.int32).contiguous()
    st = torch.cuda.current_stream().cuda_stream
    assert _lib.lib.phx_shard_gather_rows(eng.table_local_ptr(), cfg.table_rows, _ptr(shuffled), shuffled.numel(),
                                          cfg.emb_size, _ptr(landing), st) == 0
    pos = where[inv].to(torch.int32).contiguous()
    torch.cuda.synchronize()
    got = _device_out(torch, cfg, B)
    eng.rank_forward_rows_device(B, *dev, _ptr(landing), pos, *got); eng.sync()
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    eng.close()


def test_sharded_ranker_world1_matches_plain_forward(torch):
    """parallel.ShardedRanker end to end in a one-rank NCCL group (collectives, IPC landing buffer, dedup and the
    copy path all run; the row traffic stays on the device): same outputs as the plain forward, for every exchange."""
    import socket
    import torch.distributed as dist
    from x_algorithm_b200.parallel import ShardedRanker
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                            device_id=torch.device("cuda", 0))
    try:
        ocfg, w, rows_fn, eng = make_pair(max_batch=8)
        cfg = eng.cfg
        for i, (exchange, dedup) in enumerate((("copy", True), ("push", False), ("a2a", True))):
            sr = ShardedRanker(eng, exchange=exchange, dedup=dedup)
            nxt = None
            for j, B in enumerate((8, 3, 8, 5)):           # prefetched and inline exchanges, both buffer sets
                dev = nxt or _device_batch(torch, po.make_batch(ocfg, B, seed=60 + 10 * i + j, ragged=B == 3))
                want, got = _device_out(torch, cfg, B), _device_out(torch, cfg, B)
                eng.rank_device(B, *dev, *want); eng.sync()
                sr.rank_device(B, *dev, *got)
                nxt = None
                if j == 1:                                   # exchange the next batch beside this forward
                    nxt = _device_batch(torch, po.make_batch(ocfg, 8, seed=99 + i, ragged=True))
                    sr.prefetch(8, *nxt)
                eng.sync()
                assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]), (exchange, B)
            sr.close()
        eng.close()
    finally:
        dist.destroy_process_group()


# ---- full value model (xai-value-model/scoring.rs:404-489) ----------------------------------------------------------

VM_HEADS = ["favorite", "reply", "retweet", "photo_expand", "video_open", "click", "open_link", "profile_click", "vqv", "share",
            "share_via_dm", "share_via_copy_link", "dwell", "quote", "quoted_click", "quoted_vqv", "follow_author",
            "not_interested", "block_author", "mute_author", "report", "not_dwelled", "post_unexplored", "post_video",
            "grok_analyze"]
VM_CONTS = ["dwell_time", "click_dwell_time", "home_video_continuation_secs", "home_profile_visit_secs"]


def _vm_run(torch, wt, requests, contexts):
    """Run the kernel and the oracle on the same requests (lists of po.ScoringCandidate, one context each).  The kernel
    reads f32 log-probabilities, so the oracle is given exp(f64(f32(ln p))) - the wire conversion - as its
    probabilities; a field a candidate lacks is probability / value 0."""
    import dataclasses
    import x_algorithm_b200.value_model as vm
    B, C = len(requests), max(len(r) for r in requests)
    V, NC = len(VM_HEADS), len(VM_CONTS)
    lp = np.full((B, C, V), -np.inf, np.float32)
    cont = np.zeros((B, C, NC), np.float32)
    auth = np.zeros((B, C), np.int64); flags = np.zeros((B, C), np.uint8)
    bonus = np.zeros((B, C), np.float64); lift = np.full((B, C), -1, np.int32)
    cached = np.full((B, C), np.nan, np.float64)
    nvalid = np.array([len(r) for r in requests], np.int32)
    ctxa = np.zeros((B, 5), np.float64)
    oracle_reqs = []
    for b, (req, ctx) in enumerate(zip(requests, contexts)):
        ctxa[b] = [ctx.effective_oon_weight, *(ctx.oon_factors or (np.nan, np.nan)), *(ctx.in_network_factors or (np.nan, np.nan))]
        oreq = []
        for i, c in enumerate(req):
            sc = {}
            for j, h in enumerate(VM_HEADS):
                if h in c.scores:
                    with np.errstate(divide="ignore"):
                        lp[b, i, j] = np.float32(np.log(c.scores[h]))
                sc[h] = float(np.exp(np.float64(lp[b, i, j])))
            for j, h in enumerate(VM_CONTS):
                cont[b, i, j] = np.float32(c.scores.get(h, 0.0)); sc[h] = float(cont[b, i, j])
            auth[b, i] = c.author_id
            flags[b, i] = ((vm.IN_NETWORK_KNOWN if c.in_network is not None else 0) | (vm.IN_NETWORK if c.in_network else 0)
                           | (vm.IS_REPLY if c.is_reply else 0) | (vm.IS_RETWEET if c.is_retweet else 0)
                           | (vm.MUTUAL_FOLLOW if c.is_mutual_follow_author else 0) | (vm.VQV_ELIGIBLE if c.vqv_eligible else 0)
                           | (vm.QUOTED_VQV_ELIGIBLE if c.quoted_vqv_eligible else 0))
            bonus[b, i] = c.author_exploration_bonus
            lift[b, i] = -1 if c.cold_start_lift_to_rank is None else c.cold_start_lift_to_rank
            if c.weighted_score is not None:
                cached[b, i] = c.weighted_score
            oreq.append(dataclasses.replace(c, scores=sc))
        po.set_user_video_continuation(oreq)
        oracle_reqs.append(oreq)
    use_cached = not np.isnan(cached[nvalid[:, None] > np.arange(C)[None]]).any()
    pw = vm.ValueModelWeights(**{f.name: getattr(wt, f.name) for f in dataclasses.fields(wt)})
    model = vm.value_model_struct(pw, VM_HEADS, VM_CONTS)
    cu = lambda a: torch.from_numpy(a).cuda()
    w_got, s_got = vm.value_scores(model, cu(lp), cu(cont), cu(auth), weighted=cu(cached) if use_cached else None,
                                   flags=cu(flags), exploration_bonus=cu(bonus), cold_start_rank=cu(lift),
                                   num_valid=cu(nvalid), context=cu(ctxa))
    torch.cuda.synchronize()
    w_got, s_got = w_got.cpu().numpy(), s_got.cpu().numpy()
    out = []
    for b, (oreq, ctx) in enumerate(zip(oracle_reqs, contexts)):
        if not use_cached:
            oreq = [dataclasses.replace(c, weighted_score=None) for c in oreq]
        w_want, s_want = po.compute_value_scores(wt, ctx, oreq)
        n = len(oreq)
        np.testing.assert_allclose(w_got[b, :n], w_want, rtol=1e-12, atol=1e-15)
        np.testing.assert_allclose(s_got[b, :n], s_want, rtol=1e-12, atol=1e-15)
        assert (s_got[b, n:] == 0).all()
        out.append((w_got[b, :n], s_got[b, :n]))
    return out


def test_value_model_kernel_known_answers(torch):
    """The known answers of xai-value-model/scoring.rs' own tests through the kernel: equal to the oracle to 1e-12 on
    the kernel's inputs, and to the reference's expected numbers to the f32 precision of the log-probabilities."""
    from tests.test_oracle_golden import value_model_kats, neutral_factor_case
    for name, wt, ctx, cands, want_w, want_s in value_model_kats():
        (w_got, s_got), = _vm_run(torch, wt, [cands], [ctx])
        np.testing.assert_allclose(s_got, want_s, rtol=2e-6, atol=1e-9, err_msg=name)
        if want_w is not None:
            np.testing.assert_allclose(w_got, want_w, rtol=2e-6, atol=1e-9, err_msg=name)
    wt, single, neutral, cands = neutral_factor_case()
    (_, a), (_, b) = _vm_run(torch, wt, [cands, cands], [single, neutral])
    np.testing.assert_allclose(a, b, rtol=1e-12)


@pytest.mark.parametrize("mode", ["weighted", "pre_offset", "multiplicative", "cached"])
def test_value_model_kernel_vs_oracle_random(torch, mode):
    """Random requests: ragged candidate counts (up to 700 per request), few authors (so author diversity bites), tied
    scores (duplicated candidates: ties rank in input order), every gate, bonus, cold-start lift and context form."""
    rng = np.random.default_rng({"weighted": 1, "pre_offset": 2, "multiplicative": 3, "cached": 4}[mode])
    w = {h: float(rng.uniform(0.0, 5.0)) for h in VM_HEADS}
    for h in ("not_interested", "block_author", "mute_author", "report", "not_dwelled"):
        w[h] = -float(rng.uniform(1.0, 100.0))
    w.update(cont_dwell_time=0.01, cont_click_dwell_time=0.02, video_continuation=0.003, user_video_continuation=0.002,
             profile_visit_secs=0.004)
    wt = po.ValueModelWeights(w=w, post_unexplored_include_out_of_network=False, bidirectional_follow_reply_weight_boost=1.5,
                              bidirectional_follow_dwell_weight_boost=0.25, enable_author_diversity=True,
                              author_diversity_decay=0.6, author_diversity_floor=0.2, oon_rescore_in_network_replies_retweets=True,
                              multiplier_pre_offset=(mode == "pre_offset"), multiplicative=(mode == "multiplicative"),
                              not_dwelled_power_exponent=-0.5, not_dwelled_power_offset=0.11, engage_bias=0.1)
    requests, contexts = [], []
    for n in (1, 2, 37, 256, 700):
        req = []
        for i in range(n):
            sc = {h: float(rng.uniform(0.0, 0.3) if h not in ("report", "block_author", "mute_author", "not_interested")
                           else rng.uniform(0.0, 0.02)) for h in VM_HEADS}
            sc.update(dwell_time=float(rng.uniform(0, 30)), click_dwell_time=float(rng.uniform(0, 10)),
                      home_video_continuation_secs=float(rng.uniform(0, 20)), home_profile_visit_secs=float(rng.uniform(0, 5)))
            req.append(po.ScoringCandidate(
                scores=sc, author_id=int(rng.integers(1, max(2, n // 4 + 1))),
                in_network=[None, True, False][int(rng.integers(0, 3))], is_reply=bool(rng.random() < 0.2),
                is_retweet=bool(rng.random() < 0.2), is_mutual_follow_author=bool(rng.random() < 0.5),
                vqv_eligible=bool(rng.random() < 0.5), quoted_vqv_eligible=bool(rng.random() < 0.5),
                author_exploration_bonus=float(rng.uniform(-0.5, 0.5)) if rng.random() < 0.3 else 0.0,
                weighted_score=float(rng.uniform(-0.0005, 3.0)) if mode == "cached" else None))
        if n >= 4:
            import dataclasses
            req[3] = dataclasses.replace(req[1])               # an exact tie: same scores, same author
            req[n // 2].cold_start_lift_to_rank = n // 3
            req[n - 1].cold_start_lift_to_rank = 0             # ignored: only the first candidate with a lift counts
        requests.append(req)
        contexts.append([po.ScoringContext(), po.ScoringContext(0.75), po.ScoringContext(0.6, po.class_factors(0.6, 0.9), None),
                         po.ScoringContext(0.8, po.class_factors(0.5, 1.1), po.class_factors(1.2, 0.7)),
                         po.ScoringContext(0.9, None, po.class_factors(1.1, 0.9))][len(contexts)])
    _vm_run(torch, wt, requests, contexts)


def test_value_model_scorer_plugin(torch):
    """The plugin over the kernel: the reference's hand-computed case (scoring.rs:498-636) through Candidate objects;
    a candidate without scores becomes an error string and the rest are still scored."""
    import x_algorithm_b200 as px
    from tests.test_oracle_golden import value_model_kats
    name, wt, ctx, cands, want_w, want_s = value_model_kats()[0]
    import dataclasses
    pw = px.ValueModelWeights(**{f.name: getattr(wt, f.name) for f in dataclasses.fields(wt)})
    scorer = px.ValueModelScorer(pw, VM_HEADS, VM_CONTS, context=(ctx.effective_oon_weight, ctx.oon_factors, ctx.in_network_factors))
    pcs = [px.Candidate(post_id=10 + i, author_id=c.author_id, phoenix_scores=dict(c.scores), in_network=c.in_network,
                        is_reply=c.is_reply, is_retweet=c.is_retweet, is_mutual_follow_author=c.is_mutual_follow_author,
                        vqv_eligible=c.vqv_eligible, quoted_vqv_eligible=c.quoted_vqv_eligible) for i, c in enumerate(cands)]
    pcs.insert(2, px.Candidate(post_id=99, author_id=7))            # no scores
    res = scorer.run(px.Query(), pcs)
    assert len(res) == 5 and isinstance(res[2], str)
    got = [r for r in res if not isinstance(r, str)]
    np.testing.assert_allclose([r.score for r in got], want_s, rtol=2e-6, atol=1e-9)
    np.testing.assert_allclose([r.weighted_score for r in got], want_w, rtol=2e-6, atol=1e-9)
    scorer.update_all(pcs, res)
    assert pcs[2].score is None and pcs[0].score == got[0].score


def test_source_plugin_dataset_windows_and_exclusions(torch):
    """PhoenixSource over dataset windows of one shard: every dataset its own top-k and served type
    (phoenix_source.rs:140, 177-186), seen posts never returned (73-98), all equal to the oracle's top-k of the
    window with the excluded posts masked."""
    import x_algorithm_b200 as px
    from x_algorithm_b200.plugin import HistoryItem
    from x_algorithm_b200.retrieval import CorpusShard, Retriever
    ocfg, w, rows_fn, tower = make_pair(max_batch=2, emb_size=128, num_candidates=0, history_len=32)
    N = 40_000
    shard = CorpusShard(N, 128, row_offset=0, max_queries=2, max_k=400)
    shard.fill_synthetic(21)
    post_ids = np.arange(1, N + 1, dtype=np.int64) * 7
    author_ids = np.arange(N, dtype=np.int64) % 97 + 1
    datasets = [("home", 0, 30_000, 50), ("home_cold", 30_000, 38_000, 20), ("zero_fav", 38_000, 40_000, 10)]
    src = px.PhoenixSource(tower, Retriever([shard]), post_ids, author_ids, datasets=datasets)
    rng = np.random.default_rng(3)
    hist = [HistoryItem(int(p), int(a), int(rng.integers(1, 9)), int(rng.integers(1, 5)))
            for p, a in zip(rng.integers(1, 1 << 40, 20), rng.integers(1, 1 << 40, 20))]
    first = src.run(px.Query(history=hist))
    assert [c.served_type for c in first] == (["ForYouPhoenixRetrieval"] * 50 + ["ForYouPhoenixRetrievalCold"] * 20 +
                                              ["ForYouPhoenixRetrievalZeroFav"] * 10)
    # oracle: the tower's own user vector against the corpus, window by window
    users = Retriever([shard]).user_vector(tower, hist).cpu().numpy()
    sc = po.corpus_scores(users, po.synthetic_corpus_rows(np.arange(N), 128, 21))
    seen = [first[0].post_id, first[3].post_id, first[55].post_id, 12345]
    got = src.run(px.Query(history=hist, seen_post_ids=seen))
    want = []
    for _, r0, r1, k in datasets:
        masked = np.where(np.isin(post_ids[r0:r1], seen)[None], -np.inf, sc[:, r0:r1])
        want += [int(post_ids[i]) for i in po.top_k(masked, k, row_offset=r0)[1][0]]
    assert [c.post_id for c in got] == want and not set(seen) & {c.post_id for c in got}
    shard.close(); tower.close()
