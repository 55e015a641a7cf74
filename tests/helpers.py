"""Shared helpers of the GPU parity tests: build an engine and the oracle from one configuration."""
import math

import numpy as np

from oracle import phoenix_oracle as po


def make_pair(max_batch=4, table_seed=7, engine_kw=None, **kw):
    """(oracle cfg, oracle weights, table-rows function, engine) for the same model."""
    import x_algorithm_b200 as px

    engine_kw = engine_kw or {}     # options of the engine alone (no counterpart in the oracle's model)
    ocfg = po.ModelConfig(**kw)
    w = po.make_weights(ocfg, 0)
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
        num_candidate_only_layers=ocfg.num_candidate_only_layers, compute=ocfg.compute, token_combine=ocfg.token_combine, action_multi_hot=ocfg.action_multi_hot, **engine_kw)
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
