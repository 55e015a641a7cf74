"""The ranking forward over the reference's batch-prep buffers as they are (RankingBatchPrep,
xai-recsys-engine/src/python.rs:1394-1404): user-prefix token, action sets as bool [B,S,V], continuous history actions,
candidate product surfaces.  Engine through the C ABI against the oracle's rank_forward_prep, whose input stage is pinned
to the reference's block_user_reduce / block_history_reduce / block_candidate_reduce by the golden fixtures."""
import numpy as np
import pytest

from helpers import assert_heads_close, make_pair, rel_l2, to_inputs
from oracle import phoenix_oracle as po

pytestmark = pytest.mark.gpu

EXTRAS = dict(action_multi_hot=True, user_prefix=True, cand_surface=True,
              hist_continuous=((0, 30.0, True), (3, 100.0, False)))


def _run(kw, B=3, ragged=True, use_ip=True, tol=2e-2, max_batch=4):
    ocfg, w, rows_fn, eng = make_pair(max_batch=max_batch, **kw)
    pb = po.make_prep_batch(ocfg, B, seed=5, ragged=ragged, use_ip=use_ip)
    want_lp, want_cont, want_lf = po.rank_forward_prep(ocfg, w, rows_fn, pb)
    got = eng.rank_prep(pb)
    valid = pb.candidate_post_hashes[:, :, 0] != 0
    assert_heads_close(got.log_probs[valid], got.continuous[valid], want_lf[valid], want_cont[valid], tol=tol, what=str(kw))
    return ocfg, eng, pb, got


@pytest.mark.parametrize("combine", ["sum", "project"])
@pytest.mark.parametrize("use_ip", [True, False])
def test_prep_forward_with_every_extra(combine, use_ip):
    _run(dict(token_combine=combine, history_len=24, **EXTRAS), use_ip=use_ip)


@pytest.mark.parametrize("extra", ["user_prefix", "cand_surface", "hist_continuous"])
@pytest.mark.parametrize("combine", ["sum", "project"])
def test_prep_forward_one_extra_at_a_time(extra, combine):
    kw = dict(action_multi_hot=True, token_combine=combine, history_len=16)
    kw[extra] = EXTRAS[extra]
    _run(kw)


def test_prep_forward_full_precision():
    """fp32 activations (summed tokens): the engine within 2e-4 of the fp32 oracle on the logits."""
    _run(dict(compute="fp32", history_len=16, **EXTRAS), tol=2e-4)


@pytest.mark.parametrize("S", [127, 128])
def test_prefix_moves_the_history_boundary(S):
    """history_len + 1 rows in front of the candidates: 128 (the last size of the resident-history attention kernels) and
    129 (the first of the streaming ones), with qk-norm, a logit cap and a candidate-only tail."""
    _run(dict(emb_size=256, num_q_heads=4, num_kv_heads=2, key_size=64, history_len=S, num_candidates=16, num_layers=3,
              num_candidate_only_layers=1, qk_norm=True, attn_logit_cap=30.0, token_combine="project", **EXTRAS),
         B=5, max_batch=8)


def test_prep_without_extras_is_the_id_path_bit_for_bit():
    """No extras configured: the batch-prep entry point (hashed rows, bool action sets) and the id entry point (ids hashed on
    the device, action sets as bit masks) are the same forward."""
    ocfg, w, rows_fn, eng = make_pair(max_batch=4, action_multi_hot=True, history_len=16)
    b = po.make_batch(ocfg, 4, seed=5, ragged=True)
    pb = po.make_prep_batch(ocfg, 4, seed=5, ragged=True)
    a, c = eng.rank(to_inputs(b)), eng.rank_prep(pb)
    assert np.array_equal(a.log_probs, c.log_probs) and np.array_equal(a.continuous, c.continuous)


def test_prep_device_pointers_equal_host_buffers():
    import torch
    ocfg, eng, pb, got = _run(dict(token_combine="project", history_len=16, **EXTRAS))
    dev = torch.device("cuda", 0)

    class D:
        pass
    d = D()
    for name, _ in eng._PREP_FIELDS:
        a = getattr(pb, name)
        setattr(d, name, None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(dev))
    B = pb.history_post_hashes.shape[0]
    lp = torch.empty((B, ocfg.num_candidates, ocfg.num_actions), dtype=torch.float32, device=dev)
    cont = torch.empty((B, ocfg.num_candidates, ocfg.num_continuous), dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    eng.rank_prep_device(B, d, lp, cont)
    eng.sync()
    assert np.array_equal(lp.cpu().numpy(), got.log_probs) and np.array_equal(cont.cpu().numpy(), got.continuous)


def test_padded_user_is_not_attended():
    """user_hashes[b, 0] == 0 marks the prefix token as padding (recsys_model.py:1925): whatever rows the remaining user
    and IP hashes name, the request's outputs do not change."""
    ocfg, eng, pb, got = _run(dict(token_combine="project", history_len=16, **EXTRAS))
    assert pb.user_hashes[1, 0] == 0
    pb.user_hashes[1, 1:] = 12345
    pb.user_ip_hashes[1] = 777
    again = eng.rank_prep(pb)
    assert np.array_equal(again.log_probs, got.log_probs)


def test_entry_points_refuse_what_they_cannot_serve():
    import x_algorithm_b200 as px
    ocfg, w, rows_fn, eng = make_pair(max_batch=4, history_len=16, **EXTRAS)
    b = po.make_batch(ocfg, 2, seed=5)
    with pytest.raises(px.PhoenixError, match="phx_rank_forward_prep"):
        eng.rank(to_inputs(b))
    pb = po.make_prep_batch(ocfg, 2, seed=5)
    pb.history_continuous_actions = None
    with pytest.raises(px.PhoenixError, match="null input array"):
        eng.rank_prep(pb)
    # an engine whose actions are single ids has no use for the bool [B,S,V] buffer
    ocfg2, _, _, eng2 = make_pair(max_batch=4, history_len=16)
    pb2 = po.make_prep_batch(po.ModelConfig(history_len=16, action_multi_hot=True), 2, seed=5)
    with pytest.raises(px.PhoenixError, match="action_multi_hot"):
        eng2.rank_prep(pb2)
    with pytest.raises(px.PhoenixError):
        make_pair(max_batch=4, history_len=16, engine_kw=dict(pack_ragged=True), **EXTRAS)
