"""Shared helpers of the GPU parity tests: build an engine and the oracle from one configuration."""
import math

import numpy as np

from oracle import phoenix_oracle as po


def make_pair(max_batch=4, table_seed=7, engine_kw=None, **kw):
    """(oracle cfg, oracle weights, table-rows function, engine) for the same model."""
    import x_algorithm_b200 as px

    engine_kw = engine_kw or {}     # options of the engine alone (no counterpart in the oracle's model)
    ocfg = po.ModelConfig(**kw)
    w = po.make_prep_weights(ocfg, 0)   # make_weights plus the parameters of the batch-prep extras, when configured
    amp = 1.0 / math.sqrt(ocfg.emb_size)
    rows_fn = lambda idx: po.synthetic_table_rows(idx, ocfg.emb_size, table_seed, amp)
    pcfg = px.PhoenixConfig(
        emb_size=ocfg.emb_size, num_layers=ocfg.num_layers, num_q_heads=ocfg.num_q_heads,
        num_kv_heads=ocfg.num_kv_heads, key_size=ocfg.key_size, widening_factor=ocfg.widening_factor,
        history_len=ocfg.history_len, num_candidates=ocfg.num_candidates, max_batch=max_batch,
        num_actions=ocfg.num_actions, num_continuous=ocfg.num_continuous, num_action_types=ocfg.num_action_types,
        num_surfaces=ocfg.num_surfaces, num_hashes=ocfg.num_hashes, table_size=ocfg.table_size,
        rotary=ocfg.rotary, qk_norm=ocfg.qk_norm, primer_norm=ocfg.primer_norm, attn_logit_cap=ocfg.attn_logit_cap,
        attn_logit_cap_method=ocfg.attn_logit_cap_method, final_logit_cap=ocfg.final_logit_cap,
        rms_eps=ocfg.rms_eps, rope_base=float(ocfg.rope_base), dwell_norm_scale=ocfg.dwell_norm_scale,
        num_candidate_only_layers=ocfg.num_candidate_only_layers, compute=ocfg.compute, token_combine=ocfg.token_combine, action_multi_hot=ocfg.action_multi_hot,
        user_prefix=ocfg.user_prefix, cand_surface=ocfg.cand_surface, hist_continuous=ocfg.hist_continuous,
        hist_cont_hidden=ocfg.hist_cont_hidden, **engine_kw)
    eng = px.PhoenixEngine(pcfg, 0)
    eng.load_weights(w)
    eng.table_fill_synthetic(table_seed, amp)
    return ocfg, w, rows_fn, eng


def to_inputs(b):
    import x_algorithm_b200 as px
    return px.RankInputs(b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces, b.cand_post_ids,
                         b.cand_author_ids)


def rel_l2(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def logits_of(log_probs):
    """The logit a log-probability ln sigmoid(z) came from: z = ln p - ln(1 - p), in float64."""
    lp = np.minimum(np.asarray(log_probs, np.float64), -1e-12)
    return lp - np.log(-np.expm1(lp))


def assert_heads_close(got_lp, got_cont, want_logits, want_cont, tol=2e-2, what=""):
    """The engine's head outputs against the oracle's, measured where the error is most visible: on the LOGITS
    (recovered from the log-probabilities) and on the continuous values with their mean removed, each as relative L2
    below `tol` and with every single element within 5 * tol of the reference's RMS."""
    gl, wl = logits_of(got_lp), np.asarray(want_logits, np.float64)
    rms = float(np.sqrt(np.mean(wl ** 2)))
    err = float(np.linalg.norm(gl - wl) / max(np.linalg.norm(wl), 1e-30))
    worst = float(np.abs(gl - wl).max())
    assert err < tol, f"{what}: relative L2 of the logits {err:.3e}"
    assert worst < 5 * tol * rms, f"{what}: largest logit error {worst:.3e} (rms of the logits {rms:.3e})"
    out = dict(rel_l2_logits=err, max_abs_logit_err=worst, rms_logits=rms)
    if want_cont is not None and np.size(want_cont):
        wc = np.asarray(want_cont, np.float64)
        gc = np.asarray(got_cont, np.float64)
        m = wc.mean(axis=tuple(range(wc.ndim - 1)), keepdims=True)        # per continuous head
        dev = wc - m
        rms_c = float(np.sqrt(np.mean(dev ** 2)))
        err_c = float(np.linalg.norm(gc - wc) / max(np.linalg.norm(dev), 1e-30))
        worst_c = float(np.abs(gc - wc).max())
        assert err_c < tol, f"{what}: relative L2 of the mean-removed continuous values {err_c:.3e}"
        assert worst_c < 5 * tol * max(rms_c, 1e-30), f"{what}: largest continuous error {worst_c:.3e} (rms of the variation {rms_c:.3e})"
        out.update(rel_l2_continuous=err_c, max_abs_continuous_err=worst_c, rms_continuous_variation=rms_c)
    return out


def take_requests(b, idx):
    """The requests `idx` of a batch, as a batch of their own (requests are independent)."""
    idx = np.asarray(idx)
    return type(b)(*[np.ascontiguousarray(getattr(b, f)[idx]) for f in
                     ("hist_post_ids", "hist_author_ids", "hist_actions", "hist_surfaces", "cand_post_ids", "cand_author_ids")])


def check_topk_against_scores(s32, got_scores, got_ids, k, row_offset=0, slack=4e-6):
    """The returned top-k lists against full-precision scores s32 [B, N] of every row (fp32 dot products, not yet
    rounded).  The reference ranks by the bf16 rounding of the score, ties by lower row.  Two fp32 summation orders
    can put a score on either side of a bf16 rounding boundary, so a row whose fp32 score lies within `slack` of such a
    boundary may carry either rounding; everything else must be exact: (1) each returned score is an allowed rounding
    of its row's score, (2) the list is ordered by (score desc, row asc), (3) no row left out beats the last returned
    entry under its lower allowed rounding."""
    from oracle import phoenix_oracle as po
    s32 = np.asarray(s32, np.float32)
    B, N = s32.shape
    lo = po.bf16_round(s32 - np.float32(slack))
    hi = po.bf16_round(s32 + np.float32(slack))
    got_scores = np.asarray(got_scores, np.float32); got_ids = np.asarray(got_ids, np.int64)
    n_ambiguous = 0
    for b in range(B):
        rows = got_ids[b] - row_offset
        assert rows.min() >= 0 and rows.max() < N and np.unique(rows).size == k, f"query {b}: rows out of range or repeated"
        gs = got_scores[b]
        ok = (gs == lo[b, rows]) | (gs == hi[b, rows])
        assert ok.all(), f"query {b}: a returned score is not a bf16 rounding of its row's score"
        n_ambiguous += int((lo[b, rows] != hi[b, rows]).sum())
        later = (gs[1:] < gs[:-1]) | ((gs[1:] == gs[:-1]) & (got_ids[b, 1:] > got_ids[b, :-1]))
        assert later.all(), f"query {b}: list not ordered by (score desc, row asc)"
        left = np.ones(N, bool); left[rows] = False
        beats = left & ((lo[b] > gs[-1]) | ((lo[b] == gs[-1]) & (np.arange(N) < rows[-1])))
        assert not beats.any(), f"query {b}: row {int(np.flatnonzero(beats)[0]) + row_offset} belongs in the top-k"
    return n_ambiguous
