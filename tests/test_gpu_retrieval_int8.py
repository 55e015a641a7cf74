"""Retrieval over the int8 form of the corpus (the reference's post_q8 / post_scales table and _int8_dot_scores,
recsys_two_tower_model.py:2518-2533): integer dot products are exact, so ids AND scores must equal the oracle's
bit for bit - uploaded tables, the device-side quantiser, the sampled-pivot path, windows, masks, the exact passes."""
import numpy as np
import pytest

from oracle import phoenix_oracle as po

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch
    return torch


def _users(B, dim, seed):
    u = np.random.default_rng(seed).standard_normal((B, dim)).astype(np.float32)
    return u / np.linalg.norm(u, axis=1, keepdims=True)


def _table(N, dim, seed):
    r = np.random.default_rng(seed)
    q8 = r.integers(-127, 128, size=(N, dim), dtype=np.int8)
    q8[::97] = q8[5]                                   # equal rows: ties, broken by the lower row
    scales = (r.random(N, dtype=np.float32) * np.float32(0.01) + np.float32(1e-4)).astype(np.float32)
    scales[::97] = scales[5]
    return q8, scales


def _topk(torch, sh, users, k, window=None):
    B = users.shape[0]
    dev = torch.device("cuda", 0)
    u = torch.from_numpy(users).to(dev)
    sc = torch.empty((B, k), dtype=torch.float32, device=dev); ids = torch.empty((B, k), dtype=torch.int64, device=dev)
    torch.cuda.synchronize()
    if window is None:
        sh.topk_device(u, B, k, sc, ids)
    else:
        sh.topk_window_device(u, B, k, window[0], window[1], sc, ids)
    sh.sync()
    return sc.cpu().numpy(), ids.cpu().numpy()


@pytest.mark.parametrize("dim,N,B,k", [(64, 5000, 3, 40), (128, 70000, 20, 300), (32, 300000, 64, 100)])
def test_int8_table_topk_bit_exact(torch, dim, N, B, k):
    """Small shard (every row collected), a shard past the survivor buffer (sampled pivot), three batch widths."""
    from x_algorithm_b200.retrieval import CorpusShard
    q8, scales = _table(N, dim, 1)
    users = _users(B, dim, 2)
    sh = CorpusShard(N, dim, row_offset=1000, max_queries=64, max_k=512)
    sh.upload_int8(0, q8, scales)
    sh.set_int8(True)
    got_s, got_i = _topk(torch, sh, users, k)
    want_s, want_i = po.top_k(po.int8_corpus_scores(users, q8, scales), k, row_offset=1000)
    assert np.array_equal(got_i, want_i) and np.array_equal(got_s, want_s)
    sh.close()


def test_int8_windows_masks_and_exact_passes(torch):
    from x_algorithm_b200.retrieval import CorpusShard
    dim, N, B, k = 64, 90000, 7, 120
    q8, scales = _table(N, dim, 3)
    users = _users(B, dim, 4)
    scores = po.int8_corpus_scores(users, q8, scales)
    sh = CorpusShard(N, dim, max_queries=16, max_k=256)
    sh.upload_int8(0, q8, scales)
    sh.set_int8(True)
    lo, hi = 12345, 81234
    got_s, got_i = _topk(torch, sh, users, k, (lo, hi))
    want_s, want_i = po.top_k(scores[:, lo:hi], k, row_offset=lo)
    assert np.array_equal(got_i, want_i) and np.array_equal(got_s, want_s)
    elig = np.random.default_rng(5).random(N) < 0.3
    sh.set_mask(elig)
    got_s, got_i = _topk(torch, sh, users, k)
    masked = np.where(elig[None, :], scores, -np.inf)
    want_s, want_i = po.top_k(masked, k)
    assert np.array_equal(got_i, want_i) and np.array_equal(got_s, want_s)
    sh.set_mask(None)
    sh.set_exact(True)                                   # bisection on the key with counting scans of the int8 rows
    got_s, got_i = _topk(torch, sh, users, k)
    want_s, want_i = po.top_k(scores, k)
    assert np.array_equal(got_i, want_i) and np.array_equal(got_s, want_s) and sh.exact_runs() == 1
    sh.close()


def test_device_quantiser_follows_the_oracle_rule_and_bf16_scoring_is_untouched(torch):
    from x_algorithm_b200.retrieval import CorpusShard
    dim, N, B, k = 128, 40000, 5, 64
    sh = CorpusShard(N, dim, max_queries=16, max_k=128)
    sh.fill_synthetic(9)
    dev = torch.device("cuda", 0)
    rows = torch.empty((N, dim), dtype=torch.int16, device=dev)
    sh._check(__import__("x_algorithm_b200")._lib.lib.phx_corpus_read_device(sh._h, 0, N, int(rows.data_ptr())))
    corpus = po.bf16_from_bits(rows.cpu().numpy().view(np.uint16))
    users = _users(B, dim, 6)
    before_s, before_i = _topk(torch, sh, users, k)                      # bf16 scoring
    sh.quantize_int8()
    q8 = torch.empty((N, dim), dtype=torch.int8, device=dev); sc = torch.empty((N,), dtype=torch.float32, device=dev)
    sh.read_int8_device(0, N, q8, sc)
    want_q, want_sc = po.quantize_int8(corpus)
    assert np.array_equal(q8.cpu().numpy(), want_q) and np.array_equal(sc.cpu().numpy(), want_sc)
    sh.set_int8(True)
    got_s, got_i = _topk(torch, sh, users, k)
    want_s, want_i = po.top_k(po.int8_corpus_scores(users, want_q, want_sc), k)
    assert np.array_equal(got_i, want_i) and np.array_equal(got_s, want_s)
    # the int8 list is a close approximation of the bf16 one (rows normalised, 7-bit mantissa either way)
    overlap = np.mean([len(set(a) & set(b)) / k for a, b in zip(got_i, before_i)])
    assert overlap > 0.9
    sh.set_int8(False)
    again_s, again_i = _topk(torch, sh, users, k)
    assert np.array_equal(again_i, before_i) and np.array_equal(again_s, before_s)
    sh.close()


def test_int8_needs_rows_first(torch):
    import x_algorithm_b200 as px
    from x_algorithm_b200.retrieval import CorpusShard
    sh = CorpusShard(1000, 64, max_queries=4, max_k=16)
    with pytest.raises(px.PhoenixError, match="no int8 rows"):
        sh.set_int8(True)
    sh.close()
    odd = CorpusShard(1000, 48, max_queries=4, max_k=16)                 # dim not a multiple of 32
    with pytest.raises(px.PhoenixError, match="multiple of 32"):
        odd.quantize_int8()
    odd.close()
