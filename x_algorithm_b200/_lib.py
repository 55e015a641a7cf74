"""ctypes binding of libphoenix_b200.so (the C ABI declared in include/phoenix_b200.h).

There is no fallback: if the shared library is missing or does not load, importing this module
raises, and every operator of the package fails with it."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libphoenix_b200.so")

PHX_MAX_HASHES = 4
PHX_MAX_HIST_CONT = 4
PHX_MAX_BLEND_TERMS = 32
STATUS_NAMES = {0: "PHX_OK", 1: "PHX_E_ARG", 2: "PHX_E_CUDA", 3: "PHX_E_NCCL", 4: "PHX_E_TIMEOUT",
                5: "PHX_E_CAPACITY", 6: "PHX_E_STATE"}


class HashFamily(C.Structure):
    _fields_ = [("scales", C.c_int64 * PHX_MAX_HASHES), ("biases", C.c_int64 * PHX_MAX_HASHES),
                ("modulus", C.c_int64), ("table_size", C.c_int64), ("num_hashes", C.c_int32), ("_pad", C.c_int32)]


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "emb_size", "num_layers", "num_q_heads", "num_kv_heads", "key_size", "ffn_size", "history_len",
        "num_candidates", "max_batch", "num_actions", "num_continuous", "num_action_types", "num_surfaces",
        "rotary", "qk_norm", "primer_norm", "cap_method")] + [(n, C.c_float) for n in (
        "attn_logit_cap", "final_logit_cap", "rms_eps", "rope_base", "dwell_norm_scale")] + [
        ("user", HashFamily), ("item", HashFamily), ("author", HashFamily), ("ip", HashFamily),
        ("table_world", C.c_int32), ("table_rank", C.c_int32), ("num_candidate_only_layers", C.c_int32),
        ("compute_fp32", C.c_int32), ("token_project", C.c_int32), ("pack_ragged", C.c_int32), ("action_multi_hot", C.c_int32), ("user_prefix", C.c_int32),
        ("cand_surface", C.c_int32), ("num_hist_continuous", C.c_int32), ("hist_cont_hidden", C.c_int32),
        ("hist_cont_index", C.c_int32 * PHX_MAX_HIST_CONT), ("hist_cont_use_log", C.c_int32 * PHX_MAX_HIST_CONT),
        ("hist_cont_norm_scale", C.c_float * PHX_MAX_HIST_CONT), ("_pad3", C.c_int32)]


class BlendSpec(C.Structure):
    _fields_ = [("num_terms", C.c_int32), ("src", C.c_int32 * PHX_MAX_BLEND_TERMS),
                ("weight", C.c_double * PHX_MAX_BLEND_TERMS), ("total_sum", C.c_double), ("negative_sum", C.c_double)]


class RankBatch(C.Structure):
    _fields_ = [("batch", C.c_int32), ("_pad", C.c_int32), ("hist_post_ids", C.c_void_p),
                ("hist_author_ids", C.c_void_p), ("hist_actions", C.c_void_p), ("hist_surfaces", C.c_void_p),
                ("cand_post_ids", C.c_void_p), ("cand_author_ids", C.c_void_p)]


class RankBatchPrep(C.Structure):   # phx_rank_batch_prep: the reference's batch-prep buffers under its names
    _fields_ = [("batch", C.c_int32), ("_pad", C.c_int32)] + [(n, C.c_void_p) for n in (
        "user_hashes", "user_ip_hashes", "history_post_hashes", "history_auth_hashes", "history_product_surfaces",
        "history_actions", "history_continuous_actions", "candidate_post_hashes", "candidate_auth_hashes",
        "candidate_product_surfaces")]


# phx_rank_batch_hashed: the same layout with int32 [.., H] row arrays in place of the int64 id arrays
RankBatchHashed = RankBatch


class RankOut(C.Structure):
    _fields_ = [("log_probs", C.c_void_p), ("continuous", C.c_void_p), ("scores", C.c_void_p)]


class ValueModel(C.Structure):   # phx_value_model
    _fields_ = [("src", C.c_int32 * 32), ("w", C.c_double * 30), ("reply_boost", C.c_double), ("dwell_boost", C.c_double),
                ("author_diversity_decay", C.c_double), ("author_diversity_floor", C.c_double),
                ("not_dwelled_power_exponent", C.c_double), ("not_dwelled_power_offset", C.c_double),
                ("engage_bias", C.c_double), ("offset_total_sum", C.c_double), ("offset_negative_sum", C.c_double),
                ("post_unexplored_include_oon", C.c_int32), ("enable_author_diversity", C.c_int32),
                ("oon_rescore_in_network_replies_retweets", C.c_int32), ("multiplier_pre_offset", C.c_int32),
                ("multiplicative", C.c_int32), ("_pad", C.c_int32)]


class ValueInputs(C.Structure):  # phx_value_inputs
    _fields_ = [("batch", C.c_int32), ("num_candidates", C.c_int32), ("num_actions", C.c_int32),
                ("num_continuous", C.c_int32)] + [(n, C.c_void_p) for n in (
        "log_probs", "continuous", "weighted", "author_ids", "flags", "exploration_bonus", "cold_start_rank",
        "num_valid", "context")]


class DppConfig(C.Structure):   # phx_dpp_config
    _fields_ = [("top_k", C.c_int32), ("max_selected_rank", C.c_int32), ("greedy_order", C.c_int32), ("window_on", C.c_int32),
                ("theta", C.c_double), ("window_size", C.c_int32), ("_pad", C.c_int32), ("half_distance", C.c_double),
                ("sid_lambda", C.c_double)]


class DppInputs(C.Structure):   # phx_dpp_inputs
    _fields_ = [("batch", C.c_int32), ("num_candidates", C.c_int32), ("emb_dim", C.c_int32), ("num_context", C.c_int32)] + [
        (n, C.c_void_p) for n in ("scores", "embeddings", "norms", "missing", "l1", "num_valid", "ctx_embeddings", "ctx_norms",
                                  "ctx_missing", "ctx_l1", "num_context_valid")] + [("has_seed", C.c_int32), ("_pad", C.c_int32)]


class AdmissionConfig(C.Structure):   # phx_admission_config
    _fields_ = [("enabled", C.c_int32), ("eta_model", C.c_int32), ("batch_size", C.c_uint64), ("margin_us", C.c_uint64),
                ("post_us", C.c_uint64), ("fallback_budget_us", C.c_uint64), ("pipeline_depth", C.c_uint64),
                ("ewma_alpha", C.c_double)]


# every symbol include/phoenix_b200.h declares: name -> (restype, argtypes)
_P = C.c_void_p
SIGNATURES = {
    "phx_engine_create": (C.c_int32, [C.POINTER(ModelConfig), C.c_int32, C.POINTER(_P)]),
    "phx_engine_destroy": (None, [_P]),
    "phx_last_error": (C.c_char_p, [_P]),
    "phx_global_error": (C.c_char_p, []),
    "phx_load_param": (C.c_int32, [_P, C.c_char_p, _P, C.c_int64, C.c_int64]),
    "phx_table_upload": (C.c_int32, [_P, C.c_int64, C.c_int64, _P]),
    "phx_table_fill_synthetic": (C.c_int32, [_P, C.c_uint32, C.c_float]),
    "phx_set_blend": (C.c_int32, [_P, C.POINTER(BlendSpec)]),
    "phx_table_ipc_handle": (C.c_int32, [_P, _P]),
    "phx_table_attach_peer": (C.c_int32, [_P, C.c_int32, _P]),
    "phx_table_local_ptr": (C.c_int32, [_P, C.POINTER(_P)]),
    "phx_table_attach_peer_ptr": (C.c_int32, [_P, C.c_int32, _P]),
    "phx_rank_forward": (C.c_int32, [_P, C.POINTER(RankBatch), C.POINTER(RankOut)]),
    "phx_rank_rows_device": (C.c_int32, [_P, C.POINTER(RankBatch), _P, _P]),
    "phx_rank_forward_rows_device": (C.c_int32, [_P, C.POINTER(RankBatch), _P, _P, C.POINTER(RankOut)]),
    "phx_rank_submit": (C.c_int32, [_P, C.POINTER(RankBatch), C.c_int32]),
    "phx_rank_collect": (C.c_int32, [_P, C.c_int32, C.POINTER(RankOut)]),
    "phx_rank_forward_device": (C.c_int32, [_P, C.POINTER(RankBatch), C.POINTER(RankOut)]),
    "phx_value_scores_device": (C.c_int32, [C.c_int32, C.POINTER(ValueModel), C.POINTER(ValueInputs), _P, _P, _P]),
    "phx_plan_ragged": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "phx_rank_forward_packed_device": (C.c_int32, [_P, C.POINTER(RankBatch), _P, _P, C.c_int64, C.c_int64, C.POINTER(RankOut)]),
    "phx_rank_forward_hashed_device": (C.c_int32, [_P, C.POINTER(RankBatchHashed), C.POINTER(RankOut)]),
    "phx_rank_forward_hashed": (C.c_int32, [_P, C.POINTER(RankBatchHashed), C.POINTER(RankOut)]),
    "phx_rank_forward_prep_device": (C.c_int32, [_P, C.POINTER(RankBatchPrep), C.POINTER(RankOut)]),
    "phx_rank_forward_prep": (C.c_int32, [_P, C.POINTER(RankBatchPrep), C.POINTER(RankOut)]),
    "phx_rank_prefetch_device": (C.c_int32, [_P, C.POINTER(RankBatch)]),
    "phx_sync": (C.c_int32, [_P]),
    "phx_set_wait_limit_us": (C.c_int32, [_P, C.c_uint32]),
    "phx_wait_selftest": (C.c_int32, [_P]),
    "phx_dispatch_counts": (C.c_int32, [_P, C.c_int32]),
    "phx_dispatch_name": (C.c_char_p, [C.c_int32]),
    "phx_last_device_ms": (C.c_int32, [_P, C.POINTER(C.c_float)]),
    "phx_last_launch_count": (C.c_int32, [_P, C.POINTER(C.c_int32)]),
    "phx_mark": (C.c_int32, [_P, C.c_int32]),
    "phx_mark_wait": (C.c_int32, [_P, C.c_int32]),
    "phx_elapsed_ms": (C.c_int32, [_P, C.c_int32, C.c_int32, C.POINTER(C.c_float)]),
    "phx_profile_enable": (C.c_int32, [_P, C.c_int32]),
    "phx_profile_read": (C.c_int32, [_P, C.POINTER(C.c_float), C.POINTER(C.c_int32)]),
    "phx_debug_read": (C.c_int32, [_P, C.c_char_p, _P, C.c_size_t]),
    "phx_hash_ids_device": (C.c_int32, [_P, C.c_int32, _P, C.c_int64, _P]),
    "phx_shard_bucket": (C.c_int32, [_P, C.c_int64, C.c_int64, C.c_int32, _P, _P, _P, _P, _P]),
    "phx_shard_gather_rows": (C.c_int32, [_P, C.c_int64, _P, C.c_int64, C.c_int32, _P, _P]),
    "phx_shard_sum_rows": (C.c_int32, [_P, _P, C.c_int64, C.c_int32, C.c_int32, _P, _P]),
    "phx_shard_gather_push": (C.c_int32, [_P, C.c_int64, _P, C.c_int64, _P, _P, C.c_int32, C.c_int32, _P]),
    "phx_shard_dedup": (C.c_int32, [_P, C.c_int64, _P, C.c_int64, _P, _P, _P, _P]),
    "phx_shard_dedup_expand": (C.c_int32, [_P, _P, _P, C.c_int64, _P, _P]),
    "phx_copy_async": (C.c_int32, [_P, _P, C.c_uint64, _P]),
    "phx_ipc_alloc": (C.c_int32, [C.c_int32, C.c_uint64, C.POINTER(_P), _P]),
    "phx_ipc_open": (C.c_int32, [C.c_int32, _P, C.POINTER(_P)]),
    "phx_ipc_close": (C.c_int32, [_P]),
    "phx_ipc_free": (C.c_int32, [_P]),
    "phx_gather_sum_device": (C.c_int32, [_P, C.c_int32, _P, C.c_int64, _P]),
    "phx_ranker_attention_device": (C.c_int32, [C.c_int32, _P, _P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32,
                                                C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_float, C.c_int32,
                                                C.POINTER(C.c_float)]),
    "phx_gemm_device": (C.c_int32, [C.c_int32, _P, _P, _P, _P, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                    C.POINTER(C.c_float)]),
    "phx_user_tower_device": (C.c_int32, [_P, C.POINTER(RankBatch), _P]),
    "phx_corpus_create": (C.c_int32, [C.c_int32, C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.POINTER(_P)]),
    "phx_corpus_destroy": (None, [_P]),
    "phx_corpus_upload": (C.c_int32, [_P, C.c_int64, C.c_int64, _P]),
    "phx_corpus_fill_synthetic": (C.c_int32, [_P, C.c_uint32]),
    "phx_corpus_upload_int8": (C.c_int32, [_P, C.c_int64, C.c_int64, _P, _P]),
    "phx_corpus_quantize_int8": (C.c_int32, [_P]),
    "phx_corpus_set_int8": (C.c_int32, [_P, C.c_int32]),
    "phx_corpus_read_int8_device": (C.c_int32, [_P, C.c_int64, C.c_int64, _P, _P]),
    "phx_corpus_read_device": (C.c_int32, [_P, C.c_int64, C.c_int64, _P]),
    "phx_corpus_topk_device": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, _P, _P]),
    "phx_corpus_set_mask": (C.c_int32, [_P, _P]),
    "phx_corpus_topk_keys_device": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, _P]),
    "phx_topk_merge_keys_device": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "phx_corpus_set_stream": (C.c_int32, [_P, _P, C.c_int32]),
    "phx_corpus_topk_window_device": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, C.c_int64, C.c_int64, _P, _P]),
    "phx_topk_merge_device": (C.c_int32, [_P, _P, _P, C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "phx_topk_merge_static": (C.c_int32, [C.c_int32, _P, _P, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P]),
    "phx_topk_merge_static_status": (C.c_int32, [C.c_int32, _P, C.POINTER(C.c_int32)]),
    "phx_comm_unique_id": (C.c_int32, [_P]),
    "phx_comm_create": (C.c_int32, [_P, C.c_int32, C.c_int32, C.c_int32, C.POINTER(_P)]),
    "phx_comm_destroy": (None, [_P]),
    "phx_comm_last_error": (C.c_char_p, [_P]),
    "phx_comm_info": (C.c_int32, [_P, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "phx_comm_barrier": (C.c_int32, [_P, _P]),
    "phx_retrieve_topk": (C.c_int32, [_P, _P, _P, C.c_int32, C.c_int32, _P, _P, _P]),
    "phx_gather_sharded_setup": (C.c_int32, [_P, _P, C.c_int64, C.c_double]),
    "phx_gather_sum_sharded": (C.c_int32, [_P, _P, C.c_int32, _P, C.c_int64, _P, _P]),
    "phx_gather_sum_sharded_multi": (C.c_int32, [_P, _P, C.c_int32, _P, _P, _P, _P, _P]),
    "phx_gather_sharded_phase_ms": (C.c_int32, [_P, C.POINTER(C.c_float)]),
    "phx_now_us": (C.c_uint64, []),
    "phx_queue_create": (C.c_int32, [C.c_int32, C.c_int32, C.c_uint64, C.c_uint64, C.POINTER(_P)]),
    "phx_queue_destroy": (None, [_P]),
    "phx_queue_push": (C.c_int32, [_P, C.c_uint64, C.c_uint64, C.c_uint64]),
    "phx_queue_dequeue": (C.c_int32, [_P, C.c_uint64, _P, C.c_int32, C.POINTER(C.c_int32), _P, C.c_int32, C.POINTER(C.c_int32)]),
    "phx_queue_stats": (C.c_int32, [_P, C.POINTER(C.c_int32), C.POINTER(C.c_uint64)]),
    "phx_admission_create": (C.c_int32, [C.POINTER(AdmissionConfig), C.POINTER(_P)]),
    "phx_admission_destroy": (None, [_P]),
    "phx_admission_set_enabled": (C.c_int32, [_P, C.c_int32]),
    "phx_admission_reset": (C.c_int32, [_P]),
    "phx_admission_record_service_us": (C.c_int32, [_P, C.c_uint64]),
    "phx_admission_record_sojourn_us": (C.c_int32, [_P, C.c_uint64, C.c_int64]),
    "phx_admission_predicted_eta_us": (C.c_int32, [_P, C.c_int64, C.c_int32, C.POINTER(C.c_uint64)]),
    "phx_admission_should_reject": (C.c_int32, [_P, C.c_int64, C.c_int64]),
    "phx_admission_estimates": (C.c_int32, [_P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "phx_dpp_rescore_device": (C.c_int32, [C.c_int32, C.POINTER(DppConfig), C.POINTER(DppInputs), _P, _P, _P, _P]),
    "phx_corpus_sync": (C.c_int32, [_P]),
    "phx_corpus_finish": (C.c_int32, [_P, C.POINTER(C.c_int32)]),
    "phx_corpus_set_exact": (C.c_int32, [_P, C.c_int32]),
    "phx_corpus_exact_runs": (C.c_int32, [_P, C.POINTER(C.c_int64)]),
    "phx_corpus_last_device_ms": (C.c_int32, [_P, C.POINTER(C.c_float)]),
    "phx_corpus_last_error": (C.c_char_p, [_P]),
}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m x_algorithm_b200.build` (nvcc, sm_100a). "
        "This package has no CPU or PyTorch fallback.")

lib = C.CDLL(LIB_PATH)
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = the library does not export a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


class PhoenixError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message
