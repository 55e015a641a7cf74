"""Seeded synthetic weights and request batches for benchmarks of the engine (no dataset is involved: ids are
Zipf or uniform over [1, 2^40), weights N(0, 0.02) rounded to bf16).  The generators draw from the same streams, in
the same order, as the test oracle's, so a benchmark and a parity test that name the same seed see the same model
and the same requests."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bf16 -> float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)


def zipf_ids(shape, rng: np.random.Generator, s: float = 1.1) -> np.ndarray:
    """Zipf(s) ranks over [1, 2^40) by inverse CDF, scattered through an odd-multiplier bijection so that hot ids do
    not sit next to each other; never 0 (the padding id)."""
    u = rng.random(shape)
    a, n = 1.0 - s, float(1 << 40)
    rank = np.clip(np.floor(((n ** a - 1.0) * u + 1.0) ** (1.0 / a)).astype(np.int64), 1, (1 << 40) - 1)
    with np.errstate(over="ignore"):
        ids = (rank * np.int64(0x9E3779B97F4A7C15 - (1 << 64))) & np.int64((1 << 40) - 1)
    return np.where(ids == 0, 1, ids).astype(np.int64)


def make_weights(cfg, seed: int = 0, std: float = 0.02) -> Dict[str, np.ndarray]:
    """Dense parameters of a PhoenixConfig-shaped model: matrices N(0, std), norm gains 1 + N(0, 0.05), all rounded to
    bf16 (the engine reads parameters as bf16)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    D, F = cfg.emb_size, cfg.ffn_size
    QW = (cfg.num_q_heads + 2 * cfg.num_kv_heads) * cfg.key_size
    HD = cfg.num_q_heads * cfg.key_size

    def mat(*shape):
        return bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))

    def gain(n):
        return bf16_round(np.float32(1.0) + rng.standard_normal(n, dtype=np.float32) * np.float32(0.05))

    w: Dict[str, np.ndarray] = {}
    w["action_table"] = bf16_round(rng.standard_normal((cfg.num_action_types + 1, D), dtype=np.float32) / np.float32(math.sqrt(D)))
    if cfg.action_multi_hot:
        w["action_table"] = w["action_table"][1:2]
    w["surface_table"] = bf16_round(rng.standard_normal((cfg.num_surfaces + 1, D), dtype=np.float32) / np.float32(math.sqrt(D)))
    for l in range(cfg.num_layers):
        p = f"layer{l}."
        w[p + "pre_attn_norm"] = gain(D)
        w[p + "w_qkv"] = mat(D, QW)
        if cfg.qk_norm:
            w[p + "q_norm"] = gain(HD)
            w[p + "k_norm"] = gain(cfg.num_kv_heads * cfg.key_size)
        w[p + "w_out"] = mat(HD, D)
        if cfg.primer_norm:
            w[p + "post_attn_norm"] = gain(D)
            w[p + "post_ffn_norm"] = gain(D)
        w[p + "pre_ffn_norm"] = gain(D)
        w[p + "w_up"] = mat(D, F)
        w[p + "w_down"] = mat(F, D)
    w["final_norm"] = gain(D)
    w["unembed"] = mat(D, cfg.num_actions)
    w["cont_unembed"] = mat(D, cfg.num_continuous)
    if cfg.token_combine == "project":
        H2 = 2 * cfg.num_hashes
        w["proj_hist"] = bf16_round(rng.standard_normal(((H2 + 2) * D, D), dtype=np.float32) / np.float32(math.sqrt(D)))
        w["proj_cand"] = bf16_round(rng.standard_normal((H2 * D, D), dtype=np.float32) / np.float32(math.sqrt(D)))
    return w


@dataclass
class SyntheticBatch:
    hist_post_ids: np.ndarray      # int64 [B,S]   0 = padding
    hist_author_ids: np.ndarray    # int64 [B,S]
    hist_actions: np.ndarray       # int32 [B,S]
    hist_surfaces: np.ndarray      # int32 [B,S]
    cand_post_ids: np.ndarray      # int64 [B,C]
    cand_author_ids: np.ndarray    # int64 [B,C]


def make_batch(cfg, batch: int, seed: int = 2, zipf_s: Optional[float] = None, ragged: bool = False) -> SyntheticBatch:
    """One request batch: ids uniform (or Zipf(zipf_s)) over [1, 2^40); history front-filled and zero-padded at the
    tail.  ragged: valid history length uniform in [0, S], candidates in [1, C]; request 0 stays full, request 1 has
    no history and one candidate."""
    rng = np.random.Generator(np.random.PCG64(seed))
    S, C = cfg.history_len, cfg.num_candidates

    def draw(shape):
        if zipf_s is None:
            return rng.integers(1, 1 << 40, size=shape, dtype=np.int64)
        return zipf_ids(shape, rng, zipf_s)

    b = SyntheticBatch(
        hist_post_ids=draw((batch, S)), hist_author_ids=draw((batch, S)),
        hist_actions=(rng.integers(0, 1 << cfg.num_action_types, size=(batch, S)) * (rng.random((batch, S)) < 0.9)).astype(np.int32)
        if cfg.action_multi_hot else rng.integers(1, cfg.num_action_types + 1, size=(batch, S)).astype(np.int32),
        hist_surfaces=rng.integers(1, cfg.num_surfaces + 1, size=(batch, S)).astype(np.int32),
        cand_post_ids=draw((batch, C)), cand_author_ids=draw((batch, C)),
    )
    if ragged:
        hl = rng.integers(0, S + 1, size=batch)
        cl = rng.integers(1, C + 1, size=batch)
        hl[0], cl[0] = S, C
        if batch > 1:
            hl[1], cl[1] = 0, 1
        for i in range(batch):
            b.hist_post_ids[i, hl[i]:] = 0; b.hist_author_ids[i, hl[i]:] = 0
            b.hist_actions[i, hl[i]:] = 0; b.hist_surfaces[i, hl[i]:] = 0
            b.cand_post_ids[i, cl[i]:] = 0; b.cand_author_ids[i, cl[i]:] = 0
    return b


def make_blend_weights(head_names, seed: int = 1) -> Dict[str, float]:
    """A fixed blend weight per head from `seed`: positive heads uniform in [0, 5), negative heads in (-100, -1], the
    continuous dwell-time weight in [0, 0.01) under the key "cont_dwell_time"."""
    rng = np.random.Generator(np.random.PCG64(seed))
    neg = {"not_interested", "block_author", "mute_author", "report", "not_dwelled"}
    out: Dict[str, float] = {}
    for n in head_names:
        out[n] = float(-rng.uniform(1.0, 100.0)) if n in neg else float(rng.uniform(0.0, 5.0))
    out["cont_dwell_time"] = float(rng.uniform(0.0, 0.01))
    return out
