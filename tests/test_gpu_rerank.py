"""Diversity rerank (phx_dpp_rescore_device) against the oracle's restatement of vm-ranker/dpp.rs: the reference's own
unit-test cases, then random requests in every mode."""
import numpy as np
import pytest

from oracle import phoenix_oracle as po

pytestmark = pytest.mark.gpu


def _item(i, s, e, **kw):
    e16 = np.asarray(e, np.float32).astype(np.float16)
    return po.DppItem(i, float(s), e16, float(np.sqrt(np.sum(e16.astype(np.float32) ** 2, dtype=np.float32))), **kw)


def _run(torch, requests, contexts, cfg, has_seed):
    """requests: list of lists of DppItem (ids = input positions); contexts: list of lists (seed first if has_seed)."""
    from x_algorithm_b200.rerank import dpp_rescore
    B = len(requests)
    Cn = max(len(r) for r in requests)
    E = len(requests[0][0].embedding)
    Hc = max([len(c) for c in contexts] + [0])
    sc = np.zeros((B, Cn)); emb = np.zeros((B, Cn, E), np.float16); nr = np.zeros((B, Cn))
    ms = np.zeros((B, Cn), np.uint8); l1 = np.full((B, Cn), -1, np.int32); nv = np.zeros(B, np.int32)
    ce = np.zeros((B, max(Hc, 1), E), np.float16); cn = np.zeros((B, max(Hc, 1))); cm = np.zeros((B, max(Hc, 1)), np.uint8)
    cl = np.full((B, max(Hc, 1)), -1, np.int32); ncv = np.zeros(B, np.int32)
    for b, (req, ctx) in enumerate(zip(requests, contexts)):
        nv[b], ncv[b] = len(req), len(ctx)
        for i, it in enumerate(req):
            sc[b, i], emb[b, i], nr[b, i], ms[b, i], l1[b, i] = it.score, it.embedding, it.norm, it.embedding_missing, -1 if it.l1 is None else it.l1
        for i, it in enumerate(ctx):
            ce[b, i], cn[b, i], cm[b, i], cl[b, i] = it.embedding, it.norm, it.embedding_missing, -1 if it.l1 is None else it.l1
    t = lambda a: torch.from_numpy(a).cuda()
    kw = dict(ctx_embeddings_f16=t(ce), ctx_norms=t(cn), ctx_missing=t(cm), ctx_l1=t(cl), num_context_valid=t(ncv)) if Hc else {}
    idx, s, cnt = dpp_rescore(cfg, t(sc), t(emb), t(nr), missing=t(ms), l1=t(l1), num_valid=t(nv), has_seed=has_seed, **kw)
    idx, s, cnt = idx.cpu().numpy(), s.cpu().numpy(), cnt.cpu().numpy()
    return [[(int(idx[b, j]), float(s[b, j])) for j in range(cnt[b])] for b in range(B)], idx, cnt


def _oracle(req, ctx, cfg, has_seed):
    seed = ctx[0] if (has_seed and ctx) else None
    hist = ctx[1:] if (has_seed and ctx) else ctx
    window = None if cfg.window_size is None else (cfg.window_size, cfg.half_distance, cfg.sid_lambda)
    return po.dpp_rescore(req, seed, hist, cfg.top_k, cfg.theta, cfg.max_selected_rank, cfg.greedy_order, window)


def test_dpp_known_answers_of_the_reference_tests():
    """vm-ranker/dpp.rs:485-735, ids re-numbered to input positions."""
    import torch
    from x_algorithm_b200.rerank import DppConfig
    run = lambda req, ctx, cfg, seed=False: _run(torch, [req], [ctx], cfg, seed)[0][0]
    assert run([_item(0, 5.0, [1, 0, 0])], [], DppConfig()) == [(0, 5.0)]                                   # single_candidate
    same = [_item(0, 10.0, [1, 0, 0]), _item(1, 5.0, [1, 0, 0]), _item(2, 1.0, [1, 0, 0])]
    assert [i for i, _ in run(same, [], DppConfig(top_k=3, max_selected_rank=10))] == [0]                    # identical_embeddings
    div = [_item(0, 10.0, [1, 0]), _item(1, 9.5, [1, 0]), _item(2, 5.0, [0, 1])]
    ids = [i for i, _ in run(div, [], DppConfig(top_k=3, max_selected_rank=10))]
    assert 2 in ids and 1 not in ids                                                                         # orthogonal_embeddings
    two = [_item(0, 10.0, [1, 0]), _item(1, 5.0, [0, 1])]
    cfg2 = DppConfig(top_k=2, max_selected_rank=10)
    assert sorted(i for i, _ in run(two, [], cfg2)) == [0, 1]
    ids = [i for i, _ in run(two, [_item(999, 0.0, [1, 0])], cfg2, seed=True)]                               # seed_suppresses_near_duplicate
    assert 0 not in ids and 1 in ids
    three = [_item(0, 10.0, [1, 0, 0]), _item(1, 5.0, [0, 1, 0])]
    assert sorted(i for i, _ in run(three, [_item(999, 0.0, [0, 0, 1])], cfg2, seed=True)) == [0, 1]         # seed_does_not_consume_top_k_budget
    go = [_item(0, 10.0, [1, 0, 0]), _item(1, 9.0, [0.8, 0, 0.6]), _item(2, 5.0, [0, 1, 0])]
    assert run(go, [], DppConfig(top_k=3)) == [(0, 10.0), (1, 9.0), (2, 5.0)]                                # greedy_order_...
    assert run(go, [], DppConfig(top_k=3, greedy_order=True)) == [(0, 10.0), (2, 9.0), (1, 5.0)]
    win = [_item(0, 10.0, [1, 0, 0, 0]), _item(1, 9.0, [1, 0, 0, 0]), _item(2, 5.0, [0, 1, 0, 0]), _item(3, 4.0, [0, 0, 1, 0]),
           _item(4, 3.0, [0, 0, 0, 1])]
    picks = lambda size, hd, req=win, ctx=[]: [i for i, _ in run(req, ctx, DppConfig(window_size=size, half_distance=hd))]
    assert picks(2, 5.0) == [0, 2, 3, 1, 4]                                                                  # window_suppresses_a_duplicate_only_inside_the_window
    assert picks(2**31 - 1, 5.0) == [0, 2, 3, 4, 1]
    assert picks(2, 0.0) == [0, 2, 3, 1, 4]
    miss = [_item(0, 10.0, [1, 0]), _item(1, 9.0, [1, 0], embedding_missing=True), _item(2, 5.0, [0, 1])]
    assert picks(1, 5.0, miss, [_item(9, 0.0, [1, 0], embedding_missing=True)]) == [0, 1, 2]                 # window_ignores_missing_embeddings


@pytest.mark.parametrize("mode", ["kernel", "kernel_seed_greedy", "window", "window_l1"])
def test_dpp_random_requests_vs_oracle(mode):
    import torch
    from x_algorithm_b200.rerank import DppConfig
    rng = np.random.default_rng(len(mode))
    B, E = 6, 48
    requests, contexts = [], []
    for b in range(B):
        n = [1, 7, 40, 130, 96, 60][b]
        centers = rng.standard_normal((5, E))
        req = []
        for i in range(n):
            e = centers[rng.integers(5)] + 0.3 * rng.standard_normal(E)
            if mode != "kernel" and i % 9 == 4:
                e = req[i - 1].embedding.astype(np.float32)                      # exact duplicates
            req.append(_item(i, float(np.round(rng.uniform(0, 10), 1)), e / np.linalg.norm(e) * rng.uniform(0.5, 2.0),
                             embedding_missing=bool(mode.startswith("window") and rng.random() < 0.1),
                             l1=int(rng.integers(4)) if mode == "window_l1" else None))
        requests.append(req)
        nctx = {"kernel": 0, "kernel_seed_greedy": 1, "window": int(rng.integers(0, 6)), "window_l1": int(rng.integers(1, 9))}[mode]
        contexts.append([_item(1000 + j, 0.0, centers[rng.integers(5)] + 0.2 * rng.standard_normal(E),
                               l1=int(rng.integers(4)) if mode == "window_l1" else None) for j in range(nctx)])
    cfg = {"kernel": DppConfig(top_k=20, theta=0.7, max_selected_rank=50),
           "kernel_seed_greedy": DppConfig(top_k=15, theta=0.9, max_selected_rank=96, greedy_order=True),
           "window": DppConfig(top_k=25, theta=0.6, max_selected_rank=60, window_size=4, half_distance=2.0),
           "window_l1": DppConfig(top_k=30, theta=0.5, max_selected_rank=80, window_size=2**31 - 1, half_distance=3.0, sid_lambda=0.3)}[mode]
    has_seed = mode == "kernel_seed_greedy"
    got, idx, cnt = _run(torch, requests, contexts, cfg, has_seed)
    for b in range(B):
        want = _oracle(requests[b], contexts[b], cfg, has_seed)
        assert [i for i, _ in got[b]] == [i for i, _ in want], (mode, b)
        assert [s for _, s in got[b]] == [s for _, s in want], (mode, b)
        assert (idx[b, cnt[b]:] == -1).all()
