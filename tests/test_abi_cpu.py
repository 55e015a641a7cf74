"""No-GPU checks of the boundary: the shared library loads and exports every symbol the header declares,
struct layouts match the header, host-side mirrors behave like the reference's traits."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "phoenix_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(phx_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as ge
    ge.build()
    from x_algorithm_b200 import _lib
    syms = _header_symbols()
    assert len(syms) >= 25
    for s in syms:
        assert hasattr(_lib.lib, s), f"{s} declared in the header but not exported"
        assert s in _lib.SIGNATURES, f"{s} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == syms


def test_struct_layouts_match_header():
    from x_algorithm_b200 import _lib
    assert C.sizeof(_lib.HashFamily) == 8 * 4 + 8 * 4 + 8 + 8 + 4 + 4
    assert C.sizeof(_lib.ModelConfig) == 17 * 4 + 5 * 4 + 4 * C.sizeof(_lib.HashFamily) + (8 + 3 + 3 * 4 + 1) * 4
    assert C.sizeof(_lib.RankBatchPrep) == 8 + 10 * 8
    assert C.sizeof(_lib.BlendSpec) == 8 + 32 * 4 + 32 * 8 + 16 - 4 + 4   # int + pad, src, weight, two doubles
    assert C.sizeof(_lib.RankBatch) == 8 + 6 * 8 and C.sizeof(_lib.RankOut) == 24
    # phx_value_model: 32 int sources, 30 + 9 doubles, 6 ints; phx_value_inputs: 4 ints + 9 pointers
    assert C.sizeof(_lib.ValueModel) == 32 * 4 + 39 * 8 + 6 * 4 and C.sizeof(_lib.ValueInputs) == 4 * 4 + 9 * 8
    assert _lib.ModelConfig.pack_ragged.offset == C.sizeof(_lib.ModelConfig) - (3 + 3 + 3 * 4 + 1) * 4


def test_config_options_reach_the_c_struct():
    import x_algorithm_b200 as px
    c = px.PhoenixConfig(num_candidate_only_layers=2, compute="fp32", token_combine="project", pack_ragged=True).to_c()
    assert (c.num_candidate_only_layers, c.compute_fp32, c.token_project, c.pack_ragged) == (2, 1, 1, 1)
    d = px.PhoenixConfig().to_c()
    assert (d.num_candidate_only_layers, d.compute_fp32, d.token_project, d.pack_ragged) == (0, 0, 0, 0)
    import pytest
    with pytest.raises(ValueError):
        px.PhoenixConfig(compute="fp16").to_c()
    with pytest.raises(ValueError):
        px.PhoenixConfig(token_combine="mean").to_c()
    p = px.PhoenixConfig(user_prefix=True, cand_surface=True, hist_continuous=((0, 30.0, True), (3, 60.0, False)), hist_cont_hidden=32).to_c()
    assert (p.user_prefix, p.cand_surface, p.num_hist_continuous, p.hist_cont_hidden) == (1, 1, 2, 32)
    assert list(p.hist_cont_index)[:2] == [0, 3] and list(p.hist_cont_use_log)[:2] == [1, 0] and list(p.hist_cont_norm_scale)[:2] == [30.0, 60.0]
    assert (d.user_prefix, d.cand_surface, d.num_hist_continuous) == (0, 0, 0)
    with pytest.raises(ValueError):
        px.PhoenixConfig(hist_continuous=((0, 1.0, False),) * 5).to_c()


def test_value_model_struct_mirrors_the_weights():
    """phx_value_model built from ValueModelWeights: sources by PhoenixScores field order, weights by term order, the
    offset sums of the active mode (weights.rs:99-113)."""
    import x_algorithm_b200.value_model as vm
    wt = vm.ValueModelWeights(w=dict(favorite=2.0, reply=4.0, report=-100.0, not_dwelled=-3.0, cont_dwell_time=0.1,
                                     video_continuation=0.5), bidirectional_follow_reply_weight_boost=1.0,
                              enable_author_diversity=True, author_diversity_decay=0.5, author_diversity_floor=0.25, engage_bias=0.2)
    m = vm.value_model_struct(wt, ["favorite", "report", "reply"], ["dwell_time", "home_video_continuation_secs"])
    src = list(m.src)[:29]
    assert src[vm.SCORE_FIELDS.index("favorite")] == 0 and src[vm.SCORE_FIELDS.index("report")] == 1
    assert src[vm.SCORE_FIELDS.index("reply")] == 2 and src[vm.SCORE_FIELDS.index("dwell_time")] == 3
    assert src[vm.SCORE_FIELDS.index("home_video_continuation_secs")] == 4 and src[vm.SCORE_FIELDS.index("vqv")] == -1
    w = list(m.w)
    assert w[vm.TERM_ORDER.index("favorite")] == 2.0 and w[vm.TERM_ORDER.index("dwell_time")] == 0.1
    assert w[vm.TERM_ORDER.index("video_continuation")] == 0.5 and w[vm.TERM_ORDER.index("report")] == -100.0
    assert (m.offset_total_sum, m.offset_negative_sum) == (6.0 + 103.0, 103.0)
    import dataclasses
    mm = vm.value_model_struct(dataclasses.replace(wt, multiplicative=True), ["favorite"], [])
    assert (mm.offset_total_sum, mm.offset_negative_sum) == (6.0 + 0.2 + 100.0, 100.0) and mm.multiplicative == 1


def test_config_matches_oracle_layout():
    import x_algorithm_b200 as px
    from oracle import phoenix_oracle as po
    for h in (2, 4):
        cfg = px.PhoenixConfig(num_hashes=h, table_size=1 << 14)
        lay = po.ModelConfig(num_hashes=h, table_size=1 << 14).hash_layout()
        for got, want in zip(cfg.families(), (lay.user, lay.item, lay.author, lay.ip)):
            assert list(got.scales) == list(want.scales) and list(got.biases) == list(want.biases)
            assert got.modulus == want.modulus and got.table_size == want.table_size
        assert cfg.table_rows == lay.total_rows
    assert px.PhoenixConfig(emb_size=512).ffn_size == 2048 == po.ModelConfig(emb_size=512).ffn_size


def test_blend_spec_matches_oracle():
    import x_algorithm_b200 as px
    from oracle import phoenix_oracle as po
    ow = po.make_blend_weights(1)
    ospec = po.blend_spec_from_weights(ow, po.HEAD_NAMES_19, 19)
    spec = px.blend_spec_from_weights(px.ValueModelWeights(w=dict(ow.w)), px.HEAD_NAMES_19, 19)
    assert spec.num_terms == len(ospec.src) == 20
    assert list(spec.src[:20]) == ospec.src.tolist() and list(spec.weight[:20]) == ospec.weight.tolist()
    assert spec.total_sum == ospec.total_sum and spec.negative_sum == ospec.negative_sum
    assert px.HEAD_NAMES_19 == po.HEAD_NAMES_19


class _FakeEngine:
    """Stands in for the native engine: deterministic outputs, optional failure."""

    def __init__(self, cfg, fail=False):
        self.cfg, self.fail, self.calls = cfg, fail, 0

    def rank(self, inp):
        import x_algorithm_b200 as px
        self.calls += 1
        if self.fail:
            raise px.PhoenixError(2, "device lost")
        B, Cn = inp.cand_post_ids.shape
        lp = np.log(np.clip((inp.cand_post_ids % 97 + 1)[..., None] / 100.0 * np.ones(self.cfg.num_actions), 1e-6, 1)).astype(np.float32)
        cont = (inp.cand_author_ids % 30)[..., None].astype(np.float32)
        return px.RankOutputs(lp, cont, (inp.cand_post_ids % 97 + 1) / 100.0 + 0.001)


def test_scorer_contract_mirrors_reference_trait():
    import x_algorithm_b200 as px
    from x_algorithm_b200.plugin import HistoryItem
    cfg = px.PhoenixConfig(num_candidates=4, max_batch=2, history_len=3)
    sc = px.PhoenixScorer(_FakeEngine(cfg), px.HEAD_NAMES_19)
    hist = [HistoryItem(10 + i, 20 + i, 1, 1) for i in range(5)] + [HistoryItem(0, 5, 1, 1)]
    q = px.Query(user_id=1, history=hist)
    cands = [px.Candidate(post_id=100 + i, author_id=7 + i) for i in range(11)]   # 3 chunks -> 2 engine calls
    res = sc.run(q, cands)
    assert len(res) == 11 and all(not isinstance(r, str) for r in res)
    assert [r.post_id for r in res] == [c.post_id for c in cands]                 # order and length preserved
    assert sc.engine.calls == 2
    assert abs(res[0].phoenix_scores["favorite"] - ((100 % 97 + 1) / 100.0)) < 1e-6
    sc.update_all(cands, res)
    assert cands[3].weighted_score == res[3].weighted_score and cands[3].phoenix_scores is res[3].phoenix_scores
    # most recent S history items, zero entries dropped
    inp = sc._inputs(q, [cands[:4]])
    assert inp.hist_post_ids[0].tolist() == [12, 13, 14]
    # engine failure -> an error string for every candidate, no exception (phoenix_scorer.rs:131-134)
    bad = px.PhoenixScorer(_FakeEngine(cfg, fail=True), px.HEAD_NAMES_19)
    res = bad.run(q, cands)
    assert len(res) == 11 and all(isinstance(r, str) and "Phoenix prediction failed" in r for r in res)
    before = [c.weighted_score for c in cands]
    bad.update_all(cands, res)
    assert [c.weighted_score for c in cands] == before                            # only Ok results are applied
    # missing scoring sequence -> default candidates (phoenix_scorer.rs:107-109)
    res = sc.run(px.Query(history=None), cands)
    assert len(res) == 11 and all(r.phoenix_scores is None for r in res)
    assert not sc.enable(px.Query(has_cached_posts=True)) and not sc.enable(px.Query(kill_switch=True))

    class Short(px.PhoenixScorer):
        def score(self, query, candidates):
            return super().score(query, candidates)[:-1]

    res = Short(_FakeEngine(cfg), px.HEAD_NAMES_19).run(q, cands)                 # scorer.rs:29-44
    assert res == ["Scorer length_mismatch expected=11 got=10"] * 11


def test_source_contract():
    import x_algorithm_b200 as px

    class FakeRetriever:
        def retrieve_for_history(self, tower, history, k):
            return np.array([0.9, 0.8, 0.7], np.float32), np.array([2, 0, 1])

    src = px.PhoenixSource(None, FakeRetriever(), np.array([11, 0, 33]), np.array([1, 2, 3]))
    out = src.run(px.Query(history=[]))
    assert [(c.post_id, c.author_id) for c in out] == [(33, 3), (11, 1)]          # row with post id 0 dropped
    assert src.run(px.Query(history=None)) == "PhoenixSource: missing retrieval_sequence"
    assert all(c.served_type == "ForYouPhoenixRetrieval" for c in out)            # phoenix_source.rs:177-186
    # seen posts are never returned (phoenix_source.rs:73-98); the list is taken deeper to make up for them
    asked = []

    class Deep(FakeRetriever):
        def retrieve_for_history(self, tower, history, k):
            asked.append(k)
            return np.array([0.9, 0.8, 0.7], np.float32), np.array([2, 0, 1])

    src = px.PhoenixSource(None, Deep(), np.array([11, 22, 33]), np.array([1, 2, 3]))
    out = src.run(px.Query(history=[], top_k=2, seen_post_ids=[33]))
    assert asked == [3] and [c.post_id for c in out] == [11, 22]
    from x_algorithm_b200.plugin import served_type_for_dataset
    assert served_type_for_dataset("home_cold") == "ForYouPhoenixRetrievalCold"
    assert served_type_for_dataset("zero_fav") == "ForYouPhoenixRetrievalZeroFav"
    assert served_type_for_dataset("ai_video_model_2day") == "ForYouPhoenixRetrievalAiVideo"
    assert served_type_for_dataset("home") == "ForYouPhoenixRetrieval"


def test_value_scores_argument_errors_are_statuses():
    """Argument checks of phx_value_scores_device come before any CUDA call: bad sizes, a missing array and a source
    column the inputs do not have are reported as statuses with a message (no GPU needed, nothing is launched)."""
    import ctypes as C
    from x_algorithm_b200 import _lib
    import x_algorithm_b200.value_model as vm
    m = vm.value_model_struct(vm.ValueModelWeights(w=dict(favorite=1.0)), ["favorite"], ["dwell_time"])
    inp = _lib.ValueInputs()
    inp.batch, inp.num_candidates, inp.num_actions, inp.num_continuous = 1, 8, 1, 1
    out = (C.c_double * 8)()
    call = lambda i, o: _lib.lib.phx_value_scores_device(0, C.byref(m), C.byref(i), None, o, None)
    assert call(inp, None) == 1                                   # no output array
    assert call(inp, out) == 1 and b"log_probs missing" in _lib.lib.phx_global_error()
    inp.num_candidates = 5000
    assert call(inp, out) == 5 and b"4096" in _lib.lib.phx_global_error()
    inp.num_candidates, inp.num_continuous = 8, 0
    dummy = (C.c_float * 8)()
    inp.log_probs = C.addressof(dummy)      # never read: the check below fails before anything is launched
    assert call(inp, out) == 1 and b"out of range" in _lib.lib.phx_global_error()
    inp.batch = -1
    assert call(inp, out) == 1


def test_plan_ragged_offsets():
    """The host-side plan of packed rows: leading non-padding slots per request, one history row kept for a request
    without history, every slot for the whole batch as soon as one request has padding in front of a valid slot."""
    from x_algorithm_b200.engine import plan_ragged
    hp = np.array([[5, 6, 7, 0], [0, 0, 0, 0], [1, 2, 3, 4]], np.int64)
    cp = np.array([[9, 0, 0], [8, 8, 8], [0, 0, 0]], np.int64)
    ho, co = plan_ragged(hp, cp)
    assert ho.tolist() == [0, 3, 4, 8] and co.tolist() == [0, 1, 4, 4]
    cp[0] = [0, 9, 0]                                   # a hole: the batch is planned over all its slots
    ho, co = plan_ragged(hp, cp)
    assert ho.tolist() == [0, 4, 8, 12] and co.tolist() == [0, 3, 6, 9]


def test_pipeline_stages_order_and_error_handling():
    """score_stage / fetch_stage keep the pipeline's rules (candidate_pipeline.rs:306-327, 497-508): disabled
    components are skipped, scorers see the updates of the scorers before them, a scorer's failed candidates keep
    their old values, failed and disabled sources contribute nothing."""
    import x_algorithm_b200 as px
    from x_algorithm_b200.plugin import Scorer, Source, score_stage, fetch_stage

    class AddOne(Scorer):
        def score(self, q, cands):
            return [px.Candidate(score=(c.score or 0.0) + 1.0) if c.post_id != 13 else "boom" for c in cands]
        def update(self, c, s):
            c.score = s.score

    class Double(AddOne):
        def score(self, q, cands):
            return [px.Candidate(score=(c.score or 0.0) * 2.0) for c in cands]

    class Off(AddOne):
        def enable(self, q):
            return False

    cands = [px.Candidate(post_id=1, score=1.0), px.Candidate(post_id=13, score=5.0)]
    score_stage(px.Query(), cands, [AddOne(), Off(), Double()])
    assert [c.score for c in cands] == [4.0, 10.0]          # (1 + 1) * 2; the failed one skipped AddOne only

    class Src(Source):
        def __init__(self, out, on=True):
            self.out, self.on = out, on
        def enable(self, q):
            return self.on
        def source(self, q):
            return self.out

    got = fetch_stage(px.Query(), [Src([px.Candidate(post_id=1)]), Src("PhoenixSource: down"), Src([]),
                                   Src([px.Candidate(post_id=9)], on=False), Src([px.Candidate(post_id=2)])])
    assert [c.post_id for c in got] == [1, 2]


def test_header_compiles_as_c_and_matches_the_ctypes_structs(tmp_path):
    """include/phoenix_b200.h is plain C (what a cgo / FFI binding would include): a probe compiled with gcc prints the
    size of every struct and the offsets of marker fields, and they equal the ctypes mirrors of x_algorithm_b200/_lib.py."""
    import shutil
    import subprocess
    from x_algorithm_b200 import _lib
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    probes = [("phx_hash_family", _lib.HashFamily, ["num_hashes"]),
              ("phx_model_config", _lib.ModelConfig, ["user", "ip", "table_world", "num_candidate_only_layers", "compute_fp32",
                                                      "token_project", "pack_ragged", "action_multi_hot"]),
              ("phx_blend_spec", _lib.BlendSpec, ["src", "weight", "total_sum"]),
              ("phx_rank_batch", _lib.RankBatch, ["hist_post_ids", "cand_author_ids"]),
              ("phx_rank_out", _lib.RankOut, ["scores"]),
              ("phx_value_model", _lib.ValueModel, ["w", "reply_boost", "offset_total_sum", "post_unexplored_include_oon", "multiplicative"]),
              ("phx_value_inputs", _lib.ValueInputs, ["log_probs", "author_ids", "context"])]
    lines = []
    for cname, _, fields in probes:
        lines.append(f'printf("{cname} %zu", sizeof({cname}));')
        for f in fields:
            lines.append(f'printf(" %zu", offsetof({cname}, {f}));')
        lines.append('printf("\\n");')
    src = tmp_path / "probe.c"
    src.write_text("#include <stdio.h>\n#include <stddef.h>\n#include \"phoenix_b200.h\"\nint main(void) {\n" + "\n".join(lines) +
                   "\nprintf(\"hashed %zu\\n\", sizeof(phx_rank_batch_hashed));\nreturn 0; }\n")
    exe = tmp_path / "probe"
    subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-I", os.path.join(root, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.strip().splitlines()
    for (cname, ct, fields), line in zip(probes, out):
        got = line.split()
        assert got[0] == cname
        assert int(got[1]) == C.sizeof(ct), cname
        for f, off in zip(fields, got[2:]):
            assert int(off) == getattr(ct, f).offset, (cname, f)
    assert out[-1] == f"hashed {C.sizeof(_lib.RankBatchHashed)}"


def test_package_synthetic_generators_equal_the_oracles():
    """Benchmarks draw weights, batches and blend weights from the package's own generators; parity tests draw them
    from the oracle's.  Same seed -> same arrays, so that a benchmark's parity check compares like with like."""
    import dataclasses
    import x_algorithm_b200 as px
    from x_algorithm_b200 import synthetic
    from oracle import phoenix_oracle as po
    for kw in (dict(), dict(qk_norm=True, primer_norm=True, emb_size=256, num_q_heads=4, num_kv_heads=2, key_size=64),
               dict(token_combine="project", action_multi_hot=True)):
        ocfg = po.ModelConfig(**kw)
        pcfg = px.PhoenixConfig(**kw)
        wo, wp = po.make_weights(ocfg, 3), synthetic.make_weights(pcfg, 3)
        assert list(wo) == list(wp)
        for k in wo:
            np.testing.assert_array_equal(wo[k], wp[k], err_msg=k)
        for zs, ragged in ((None, False), (1.1, True)):
            bo, bp = po.make_batch(ocfg, 5, seed=9, zipf_s=zs, ragged=ragged), synthetic.make_batch(pcfg, 5, seed=9, zipf_s=zs, ragged=ragged)
            for f in dataclasses.fields(bo):
                np.testing.assert_array_equal(getattr(bo, f.name), getattr(bp, f.name), err_msg=f.name)
    assert synthetic.make_blend_weights(px.HEAD_NAMES_19, 1) == dict(po.make_blend_weights(1).w)
