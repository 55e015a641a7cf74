"""Host-side mirror of the value model's weights (xai-value-model/weights.rs:8-114) and the flattening
of `weighted_terms` (xai-value-model/scoring.rs:122-261) into the ordered term list the engine's fused
blend consumes.  Per-candidate eligibility gates (vqv eligibility, network membership, follow boosts)
are outside the fused path: the flattening is the all-gates-neutral case."""
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


@dataclass
class ValueModelWeights:
    w: Dict[str, float] = field(default_factory=dict)

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
