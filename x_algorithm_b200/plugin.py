"""Scorer / Source plugins over the engine, mirroring the reference's plugin traits
(candidate-pipeline/scorer.rs:9-64, candidate-pipeline/source.rs:11-42) and the two Phoenix plugins
(home-mixer/scorers/phoenix_scorer.rs:80-185, home-mixer/scorers/phoenix_scores_ranking_scorer.rs:15-35,
home-mixer/sources/phoenix_source.rs:103-150).

Contract kept from the traits: `score` returns exactly one result per candidate, in input order; a
failed engine call turns into an error string for every candidate and never raises; `run` replaces a
wrong-length result by `length_mismatch` errors; `update_all` applies only the successful results."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from ._lib import PhoenixError
from .engine import PhoenixEngine, RankInputs


@dataclass
class HistoryItem:
    post_id: int
    author_id: int
    action: int        # 1..num_action_types
    surface: int       # 1..num_surfaces


@dataclass
class Query:
    """The part of ScoredPostsQuery the Phoenix plugins read: the user's scoring sequence."""
    user_id: int = 0
    history: Optional[List[HistoryItem]] = None     # scoring_sequence / retrieval_sequence; None = absent
    has_cached_posts: bool = False
    kill_switch: bool = False
    top_k: int = 1000
    seen_post_ids: Optional[Sequence[int]] = None   # seen / served / impressed posts the source must not return


@dataclass
class Candidate:
    post_id: int = 0
    author_id: int = 0
    phoenix_scores: Optional[Dict[str, float]] = None   # head name -> probability (dwell_time: seconds)
    weighted_score: Optional[float] = None
    score: Optional[float] = None
    served_type: Optional[str] = None               # set by the source (phoenix_source.rs:177-186)
    # what the value model reads besides the scores (xai-value-model/inputs.rs:3-17, filled as in
    # home-mixer/scorers/value_model.rs:67-94)
    in_network: Optional[bool] = None
    is_reply: bool = False
    is_retweet: bool = False
    is_mutual_follow_author: bool = False
    vqv_eligible: bool = False
    quoted_vqv_eligible: bool = False
    cold_start_lift_to_rank: Optional[int] = None
    author_exploration_bonus: float = 0.0


Result = Union[Candidate, str]   # Ok(candidate) | Err(message)


class Scorer:
    def enable(self, query: Query) -> bool:
        return True

    def score(self, query: Query, candidates: Sequence[Candidate]) -> List[Result]:
        raise NotImplementedError

    def update(self, candidate: Candidate, scored: Candidate) -> None:
        raise NotImplementedError

    def run(self, query: Query, candidates: Sequence[Candidate]) -> List[Result]:
        scored = self.score(query, candidates)
        if len(scored) == len(candidates):
            return scored
        msg = f"Scorer length_mismatch expected={len(candidates)} got={len(scored)}"
        return [msg] * len(candidates)

    def update_all(self, candidates: Sequence[Candidate], scored: Sequence[Result]) -> None:
        for c, s in zip(candidates, scored):
            if not isinstance(s, str):
                self.update(c, s)


def score_stage(query: Query, candidates: List[Candidate], scorers: Sequence[Scorer]) -> List[Candidate]:
    """The scorer stage of the pipeline (candidate-pipeline/candidate_pipeline.rs:497-508): the enabled scorers one
    after another over the same candidates, each one's successful results applied before the next runs - e.g.
    [PhoenixScorer, ValueModelScorer]: probabilities first, then the value model on them."""
    for scorer in scorers:
        if not scorer.enable(query):
            continue
        scorer.update_all(candidates, scorer.run(query, candidates))
    return candidates


def fetch_stage(query: Query, sources: Sequence["Source"]) -> List[Candidate]:
    """The source stage (candidate_pipeline.rs:306-327): every enabled source, failed ones (an error string) and empty
    ones dropped, the rest concatenated in source order."""
    out: List[Candidate] = []
    for src in sources:
        if not src.enable(query):
            continue
        got = src.run(query)
        if not isinstance(got, str):
            out.extend(got)
    return out


class PhoenixScorer(Scorer):
    """Ranks one request's candidates in chunks of the engine's candidate capacity.  Fills
    `phoenix_scores` (probabilities = exp(ln p), the client-side conversion of
    home-mixer/candidate_pipeline/performance_tests.rs:516-521) and, when a blend is set on the engine,
    `weighted_score` / `score` (phoenix_scores_ranking_scorer.rs:15-35)."""

    def __init__(self, engine: PhoenixEngine, head_names: Sequence[str], cont_names: Sequence[str] = ("dwell_time",)):
        self.engine = engine
        self.head_names = list(head_names)
        self.cont_names = list(cont_names)

    def enable(self, query: Query) -> bool:
        return not query.has_cached_posts and not query.kill_switch

    def _inputs(self, query: Query, chunks: List[Sequence[Candidate]]) -> RankInputs:
        cfg = self.engine.cfg
        B, S, C = len(chunks), cfg.history_len, cfg.num_candidates
        hp = np.zeros((B, S), np.int64); ha = np.zeros((B, S), np.int64)
        act = np.zeros((B, S), np.int32); srf = np.zeros((B, S), np.int32)
        cp = np.zeros((B, C), np.int64); ca = np.zeros((B, C), np.int64)
        # most recent S items, front-filled, entries without post or author skipped
        # (phoenix/crates/common/xai-recsys/src/util.rs:1495-1503)
        hist = [h for h in (query.history or []) if h.post_id != 0 and h.author_id != 0][-S:]
        for j, h in enumerate(hist):
            hp[:, j], ha[:, j], act[:, j], srf[:, j] = h.post_id, h.author_id, h.action, h.surface
        for i, ch in enumerate(chunks):
            for j, c in enumerate(ch):
                cp[i, j], ca[i, j] = c.post_id, c.author_id
        return RankInputs(hp, ha, act, srf, cp, ca)

    def score(self, query: Query, candidates: Sequence[Candidate]) -> List[Result]:
        n = len(candidates)
        if query.history is None:                       # phoenix_scorer.rs:107-109
            return [Candidate() for _ in range(n)]
        if n == 0:
            return []
        cfg = self.engine.cfg
        C = cfg.num_candidates
        chunks = [candidates[i:i + C] for i in range(0, n, C)]
        out: List[Result] = []
        try:
            for g in range(0, len(chunks), cfg.max_batch):
                group = chunks[g:g + cfg.max_batch]
                res = self.engine.rank(self._inputs(query, group))
                probs = np.exp(res.log_probs.astype(np.float64))
                for i, ch in enumerate(group):
                    for j, c in enumerate(ch):
                        if c.post_id == 0:
                            out.append("Phoenix prediction failed: candidate without post id")
                            continue
                        ps = {name: float(probs[i, j, k]) for k, name in enumerate(self.head_names)}
                        for k, name in enumerate(self.cont_names):
                            ps[name] = float(res.continuous[i, j, k])
                        w = float(res.scores[i, j]) if res.scores is not None else None
                        out.append(Candidate(post_id=c.post_id, author_id=c.author_id, phoenix_scores=ps,
                                             weighted_score=w, score=w))
        except PhoenixError as err:                      # phoenix_scorer.rs:131-134
            return [f"Phoenix prediction failed: {err}"] * n
        return out

    def update(self, candidate: Candidate, scored: Candidate) -> None:
        candidate.phoenix_scores = scored.phoenix_scores
        if scored.weighted_score is not None:
            candidate.weighted_score = scored.weighted_score
            candidate.score = scored.score


class ValueModelScorer(Scorer):
    """The value model over candidates that already carry `phoenix_scores` (home-mixer/scorers/value_model.rs:62-103
    building the inputs, xai-value-model/scoring.rs:404-489 scoring them): one kernel launch per request,
    `weighted_score` = fuse_heads with the candidate's gates, `score` = the final value score (exploration bonus,
    cold-start lift, author diversity, out-of-network weight, class factors).  A candidate without scores gets an
    error string, the others are still scored."""

    def __init__(self, weights, head_names: Sequence[str], cont_names: Sequence[str] = ("dwell_time",), device: int = 0,
                 context: Optional[Tuple[float, Optional[Tuple[float, float]], Optional[Tuple[float, float]]]] = None):
        from .value_model import value_model_struct
        self.head_names, self.cont_names = list(head_names), list(cont_names)
        self.model = value_model_struct(weights, self.head_names, self.cont_names)
        self.device = device
        self.context = context      # (effective_oon_weight, oon factors, in-network factors) or None = defaults

    def score(self, query: Query, candidates: Sequence[Candidate]) -> List[Result]:
        import torch

        from . import value_model as vm
        n = len(candidates)
        if n == 0:
            return []
        ok = [c.phoenix_scores is not None for c in candidates]
        idx = [i for i in range(n) if ok[i]]
        if not idx:
            return ["value model: candidate without phoenix scores"] * n
        m = len(idx)
        V, NC = len(self.head_names), len(self.cont_names)
        lp = np.full((1, m, V), -np.inf, np.float32); cont = np.zeros((1, m, max(NC, 1)), np.float32)
        auth = np.zeros((1, m), np.int64); flags = np.zeros((1, m), np.uint8)
        bonus = np.zeros((1, m), np.float64); lift = np.full((1, m), -1, np.int32)
        for j, i in enumerate(idx):
            c = candidates[i]
            for k, name in enumerate(self.head_names):
                p = c.phoenix_scores.get(name)
                if p is not None and p > 0.0:
                    lp[0, j, k] = math.log(p)
            for k, name in enumerate(self.cont_names):
                cont[0, j, k] = c.phoenix_scores.get(name) or 0.0
            auth[0, j] = c.author_id
            flags[0, j] = ((vm.IN_NETWORK_KNOWN if c.in_network is not None else 0) | (vm.IN_NETWORK if c.in_network else 0)
                           | (vm.IS_REPLY if c.is_reply else 0) | (vm.IS_RETWEET if c.is_retweet else 0)
                           | (vm.MUTUAL_FOLLOW if c.is_mutual_follow_author else 0) | (vm.VQV_ELIGIBLE if c.vqv_eligible else 0)
                           | (vm.QUOTED_VQV_ELIGIBLE if c.quoted_vqv_eligible else 0))
            bonus[0, j] = c.author_exploration_bonus
            lift[0, j] = -1 if c.cold_start_lift_to_rank is None else c.cold_start_lift_to_rank
        ctx = None
        if self.context is not None:
            eow, oon, inn = self.context
            ctx = np.array([[eow, *(oon or (np.nan, np.nan)), *(inn or (np.nan, np.nan))]], np.float64)
        try:
            dev = torch.device("cuda", self.device)
            cu = lambda a: None if a is None else torch.from_numpy(a).to(dev)
            w, s = vm.value_scores(self.model, cu(lp), cu(cont[:, :, :NC]) if NC else None, cu(auth), flags=cu(flags),
                                   exploration_bonus=cu(bonus), cold_start_rank=cu(lift), context=cu(ctx), device=self.device)
            w, s = w.cpu().numpy()[0], s.cpu().numpy()[0]
        except (PhoenixError, RuntimeError) as err:
            return [f"value model failed: {err}"] * n
        out: List[Result] = ["value model: candidate without phoenix scores"] * n
        for j, i in enumerate(idx):
            c = candidates[i]
            out[i] = Candidate(post_id=c.post_id, author_id=c.author_id, weighted_score=float(w[j]), score=float(s[j]))
        return out

    def update(self, candidate: Candidate, scored: Candidate) -> None:
        candidate.weighted_score, candidate.score = scored.weighted_score, scored.score


class Source:
    def enable(self, query: Query) -> bool:
        return True

    def source(self, query: Query) -> Union[List[Candidate], str]:
        raise NotImplementedError

    def run(self, query: Query) -> Union[List[Candidate], str]:
        return self.source(query)


# dataset type of a retrieval window -> served type of its candidates (home-mixer/sources/phoenix_source.rs:177-186)
SERVED_TYPE_FOR_DATASET = {"home_cold": "ForYouPhoenixRetrievalCold", "zero_fav": "ForYouPhoenixRetrievalZeroFav",
                           "ai_video_self_2day": "ForYouPhoenixRetrievalAiVideo", "ai_video_model_2day": "ForYouPhoenixRetrievalAiVideo"}


def served_type_for_dataset(dataset: str) -> str:
    return SERVED_TYPE_FOR_DATASET.get(dataset, "ForYouPhoenixRetrieval")


class PhoenixSource(Source):
    """User tower + exhaustive top-k over the corpus shards of this process
    (home-mixer/sources/phoenix_source.rs:113-150).  `post_ids` / `author_ids` map corpus rows to ids
    like the reference's reply (phoenix/xrex/inference/model_runner.py:5332-5360); rows whose post id
    is 0 are dropped (xai-recsys-engine/src/python.rs:846-864).

    `datasets`: the retrieval datasets of the post table as (dataset type, first row, end row, top-k) - each gets its
    own top-k over its row window (the per-dataset top-k of phoenix_source.rs:140, served by slice_and_top_k,
    recsys_two_tower_model.py:2660-2686) and its candidates the dataset's served type; without it one top-k over the
    whole corpus.  Windows need a single-shard retriever.  Posts in `query.seen_post_ids` are never returned
    (seen_post_exclusions, phoenix_source.rs:73-98): the top-k is taken that many entries deeper and the excluded
    posts dropped, which equals masking them before the top-k."""

    def __init__(self, tower: PhoenixEngine, retriever, post_ids: np.ndarray, author_ids: np.ndarray,
                 datasets: Optional[Sequence[Tuple[str, int, int, int]]] = None):
        self.tower = tower
        self.retriever = retriever
        self.post_ids = post_ids
        self.author_ids = author_ids
        self.datasets = list(datasets) if datasets else None
        if self.datasets and len(getattr(retriever, "shards", ())) != 1:
            raise ValueError("PhoenixSource: dataset windows need a single-shard retriever")

    def enable(self, query: Query) -> bool:
        return not query.has_cached_posts

    def _candidates(self, scores, rows, want: int, excluded, served: str) -> List[Candidate]:
        out = []
        for s, r in zip(scores, rows):
            pid = int(self.post_ids[r])
            if pid == 0 or pid in excluded:
                continue
            out.append(Candidate(post_id=pid, author_id=int(self.author_ids[r]), score=float(s), served_type=served))
            if len(out) == want:
                break
        return out

    def source(self, query: Query) -> Union[List[Candidate], str]:
        if query.history is None:
            return "PhoenixSource: missing retrieval_sequence"
        excluded = set(int(p) for p in (query.seen_post_ids or ()))
        try:
            if not self.datasets:
                depth = query.top_k + len(excluded)
                shards = getattr(self.retriever, "shards", None)
                if shards:
                    depth = min(depth, min(sh.rows for sh in shards))
                scores, rows = self.retriever.retrieve_for_history(self.tower, query.history, depth)
                return self._candidates(scores, rows, query.top_k, excluded, served_type_for_dataset(""))
            import torch
            users = self.retriever.user_vector(self.tower, query.history)
            shard = self.retriever.shards[0]
            out: List[Candidate] = []
            for dataset, r0, r1, k in self.datasets:
                depth = min(k + len(excluded), r1 - r0)
                sc = torch.empty((1, depth), dtype=torch.float32, device=users.device)
                ids = torch.empty((1, depth), dtype=torch.int64, device=users.device)
                shard.topk_window_device(users, 1, depth, r0, r1, sc, ids)
                shard.sync()
                out += self._candidates(sc[0].cpu().numpy(), ids[0].cpu().numpy(), k, excluded, served_type_for_dataset(dataset))
            return out
        except PhoenixError as err:
            return f"PhoenixSource: {err}"
