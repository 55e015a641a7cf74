"""Host-side mirror of the value model's weights (xai-value-model/weights.rs:8-114) and the flattening
of `weighted_terms` (xai-value-model/scoring.rs:122-261) into the ordered term list the engine's fused
blend consumes.  Per-candidate eligibility gates (vqv eligibility, network membership, follow boosts)
are outside the fused path: the flattening is the all-gates-neutral case.  The full value model
(`compute_value_scores`, scoring.rs:404-489: gates, multiplicative mode, exploration bonus, cold-start
lift, author diversity, out-of-network weight, class factors) runs as its own kernel behind the heads:
`value_model_struct` + `value_scores`."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Sequence

from . import _lib

POSITIVE_FIELDS = ["favorite", "reply", "retweet", "photo_expand", "video_open", "click", "open_link",
                   "profile_click", "vqv", "share", "share_via_dm", "share_via_copy_link", "dwell", "quote",
                   "quoted_click", "quoted_vqv", "follow_author", "post_unexplored", "post_video", "grok_analyze"]
NEGATIVE_FIELDS = ["not_interested", "block_author", "mute_author", "report", "not_dwelled"]
# summation order of the reference's term array (scoring.rs:145-260)
TERM_ORDER = ["favorite", "reply", "retweet", "photo_expand", "video_open", "click", "open_link", "profile_click",
              "vqv", "share", "share_via_dm", "share_via_copy_link", "dwell", "quote", "quoted_click", "quoted_vqv",
              "dwell_time", "click_dwell_time", "video_continuation", "user_video_continuation",
              "profile_visit_secs", "follow_author", "not_interested", "block_author", "mute_author", "report",
              "not_dwelled", "post_unexplored", "post_video", "grok_analyze"]
CONT_WEIGHT_FIELD = {"dwell_time": "cont_dwell_time", "click_dwell_time": "cont_click_dwell_time"}
# the 19 discrete heads of the benchmark workload, named after the score fields they feed
# (home-mixer/side_effects/teacher_score_side_effect.rs:43-74)
HEAD_NAMES_19 = ["favorite", "reply", "retweet", "photo_expand", "video_open", "click", "open_link", "profile_click",
                 "vqv", "share", "share_via_dm", "share_via_copy_link", "dwell", "quote", "quoted_click",
                 "follow_author", "not_interested", "block_author", "report"]


# PhoenixScores fields in declaration order (xai-value-model/phoenix_scores.rs:2-32)
SCORE_FIELDS = ["favorite", "reply", "retweet", "photo_expand", "video_open", "click", "open_link", "profile_click",
                "vqv", "share", "share_via_dm", "share_via_copy_link", "dwell", "quote", "quoted_click", "quoted_vqv",
                "follow_author", "not_interested", "block_author", "mute_author", "report", "not_dwelled",
                "post_unexplored", "post_video", "grok_analyze", "dwell_time", "click_dwell_time",
                "home_video_continuation_secs", "home_profile_visit_secs"]
# CandidateScoringInputs flags (xai-value-model/inputs.rs:3-17) as bits of the per-candidate byte
IN_NETWORK_KNOWN, IN_NETWORK, IS_REPLY, IS_RETWEET, MUTUAL_FOLLOW, VQV_ELIGIBLE, QUOTED_VQV_ELIGIBLE = 1, 2, 4, 8, 16, 32, 64


@dataclass
class ValueModelWeights:
    w: Dict[str, float] = field(default_factory=dict)
    post_unexplored_include_out_of_network: bool = False
    bidirectional_follow_reply_weight_boost: float = 0.0
    bidirectional_follow_dwell_weight_boost: float = 0.0
    enable_author_diversity: bool = False
    author_diversity_decay: float = 0.0
    author_diversity_floor: float = 0.0
    oon_rescore_in_network_replies_retweets: bool = False
    multiplier_pre_offset: bool = False
    multiplicative: bool = False
    not_dwelled_power_exponent: float = 0.0
    not_dwelled_power_offset: float = 0.0
    engage_bias: float = 0.0

    def get(self, k: str) -> float:
        return float(self.w.get(k, 0.0))

    def positive_sum(self) -> float:   # weights.rs:56-77
        s = 0.0
        for k in POSITIVE_FIELDS:
            s = s + self.get(k)
        return s

    def negative_sum(self) -> float:   # weights.rs:79-85
        s = 0.0
        for k in NEGATIVE_FIELDS:
            s = s + self.get(k)
        return -s

    def total_sum(self) -> float:      # weights.rs:87-89
        return self.positive_sum() + self.negative_sum()

    def offset_negative_sum(self) -> float:   # weights.rs:91-93, 99-105
        if self.multiplicative:
            return -(self.get("not_interested") + self.get("block_author") + self.get("mute_author") + self.get("report"))
        return self.negative_sum()

    def offset_total_sum(self) -> float:      # weights.rs:95-97, 107-113
        if self.multiplicative:
            return self.positive_sum() + self.engage_bias + self.offset_negative_sum()
        return self.total_sum()


def blend_spec_from_weights(wt: ValueModelWeights, head_names: Sequence[str], num_actions: int,
                            cont_names: Sequence[str] = ("dwell_time",)) -> _lib.BlendSpec:
    spec = _lib.BlendSpec()
    n = 0
    for name in TERM_ORDER:
        if name in head_names:
            spec.src[n], spec.weight[n] = list(head_names).index(name), wt.get(name); n += 1
        elif name in cont_names:
            spec.src[n], spec.weight[n] = num_actions + list(cont_names).index(name), wt.get(CONT_WEIGHT_FIELD[name]); n += 1
    spec.num_terms = n
    spec.total_sum, spec.negative_sum = wt.total_sum(), wt.negative_sum()
    return spec


def value_model_struct(wt: ValueModelWeights, head_names: Sequence[str], cont_names: Sequence[str] = ("dwell_time",)) -> _lib.ValueModel:
    """phx_value_model for a model whose discrete heads are `head_names` (log_probs columns) and whose continuous
    heads are `cont_names`; a PhoenixScores field the model does not produce is None."""
    m = _lib.ValueModel()
    heads, conts = list(head_names), list(cont_names)
    for i in range(32):
        m.src[i] = -1
    for i, f in enumerate(SCORE_FIELDS):
        if f in heads:
            m.src[i] = heads.index(f)
        elif f in conts:
            m.src[i] = len(heads) + conts.index(f)
    for i, t in enumerate(TERM_ORDER):
        m.w[i] = wt.get(CONT_WEIGHT_FIELD.get(t, t))
    m.reply_boost, m.dwell_boost = wt.bidirectional_follow_reply_weight_boost, wt.bidirectional_follow_dwell_weight_boost
    m.author_diversity_decay, m.author_diversity_floor = wt.author_diversity_decay, wt.author_diversity_floor
    m.not_dwelled_power_exponent, m.not_dwelled_power_offset = wt.not_dwelled_power_exponent, wt.not_dwelled_power_offset
    m.engage_bias = wt.engage_bias
    m.offset_total_sum, m.offset_negative_sum = wt.offset_total_sum(), wt.offset_negative_sum()
    m.post_unexplored_include_oon = int(wt.post_unexplored_include_out_of_network)
    m.enable_author_diversity = int(wt.enable_author_diversity)
    m.oon_rescore_in_network_replies_retweets = int(wt.oon_rescore_in_network_replies_retweets)
    m.multiplier_pre_offset, m.multiplicative = int(wt.multiplier_pre_offset), int(wt.multiplicative)
    return m


def value_scores(model: _lib.ValueModel, log_probs, continuous, author_ids, *, weighted=None, flags=None,
                 exploration_bonus=None, cold_start_rank=None, num_valid=None, context=None, device: int = 0):
    """compute_value_scores (scoring.rs:404-489) on the GPU for a batch of requests.  Arguments are CUDA torch tensors:
    log_probs f32 [B,C,V], continuous f32 [B,C,NC], author_ids i64 [B,C]; optional weighted f64 [B,C] (cached weighted
    score), flags u8 [B,C], exploration_bonus f64 [B,C], cold_start_rank i32 [B,C] (-1 = none), num_valid i32 [B],
    context f64 [B,5].  Returns (weighted f64 [B,C], scores f64 [B,C]); candidates past num_valid are left untouched."""
    import ctypes as C

    import torch
    B, Cn, V = log_probs.shape
    NC = continuous.shape[2] if continuous is not None else 0
    inp = _lib.ValueInputs()
    inp.batch, inp.num_candidates, inp.num_actions, inp.num_continuous = B, Cn, V, NC
    want = dict(log_probs=(log_probs, torch.float32), continuous=(continuous, torch.float32), weighted=(weighted, torch.float64),
                author_ids=(author_ids, torch.int64), flags=(flags, torch.uint8), exploration_bonus=(exploration_bonus, torch.float64),
                cold_start_rank=(cold_start_rank, torch.int32), num_valid=(num_valid, torch.int32), context=(context, torch.float64))
    keep = []
    for name, (t, dt) in want.items():
        if t is None:
            setattr(inp, name, None)
            continue
        assert t.is_cuda and t.dtype == dt, f"value_scores: {name} must be a CUDA tensor of {dt}"
        t = t.contiguous(); keep.append(t)
        setattr(inp, name, t.data_ptr())
    w_out = torch.zeros((B, Cn), dtype=torch.float64, device=log_probs.device)
    s_out = torch.zeros((B, Cn), dtype=torch.float64, device=log_probs.device)
    stream = torch.cuda.current_stream().cuda_stream
    st = _lib.lib.phx_value_scores_device(device, C.byref(model), C.byref(inp), w_out.data_ptr(), s_out.data_ptr(), stream)
    if st != 0:
        from .engine import PhoenixError
        raise PhoenixError(st, _lib.lib.phx_global_error().decode())
    return w_out, s_out
