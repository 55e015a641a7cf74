/*
 * phoenix_b200.h - C ABI of the B200-native Phoenix inference engine.
 *
 * The library replaces everything below the in-process engine seam of the reference's serving
 * stack: the point where the model runner has a batch of featurised requests in host buffers
 * and wants log-probabilities / continuous predictions / retrieval rows back
 * (phoenix/xrex/inference/model_runner.py:3026-3146, 4141-4222, 5114-5360).  A Scorer / Source
 * plugin (candidate-pipeline/scorer.rs:9-64, candidate-pipeline/source.rs:11-42) binds these
 * entry points with `extern "C"`.
 *
 * Conventions: every call returns a phx_status (0 = ok); no exception or abort crosses the ABI;
 * the caller owns all in/out buffers; the engine owns weights, tables and work space; one engine
 * per device; calls on one engine are serialised by the caller (the reference has a single
 * dispatch thread, model_runner.py:4259).  Pointers named *_host are host memory, *_dev are
 * device memory of the engine's device.  All multi-dimensional arrays are dense row-major.
 */
#ifndef PHOENIX_B200_H_
#define PHOENIX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t phx_status;
enum {
  PHX_OK = 0,
  PHX_E_ARG = 1,      /* bad argument / unsupported configuration */
  PHX_E_CUDA = 2,     /* a CUDA call failed; see phx_last_error */
  PHX_E_NCCL = 3,
  PHX_E_TIMEOUT = 4,  /* a bounded device-side wait ran out; the context stays usable */
  PHX_E_CAPACITY = 5, /* batch / k / n exceeds what the engine was created for */
  PHX_E_STATE = 6     /* weights or tables not loaded yet */
};

#define PHX_MAX_HASHES 4
#define PHX_MAX_HIST_CONT 4
#define PHX_MAX_BLEND_TERMS 32

/* One hash family: phoenix/xrex/models/recsys_embedding.py:175-199 (HashKeys),
 * phoenix/crates/common/xai-recsys/src/model_config.rs:156-201 (hash_user_id / hash_item_id /
 * hash_author_id). */
typedef struct phx_hash_family {
  int64_t scales[PHX_MAX_HASHES];
  int64_t biases[PHX_MAX_HASHES];
  int64_t modulus;
  int64_t table_size; /* buckets; row = (raw mod (table_size-1)) + 1 + region offset */
  int32_t num_hashes;
  int32_t _pad;
} phx_hash_family;

/* Model geometry and options: TransformerConfig / RecsysAttentionConfig / RecsysModelConfig
 * (phoenix/xrex/configs/xrecsys.py:1051-1090, phoenix/xrex/models/attention.py:16-38). */
typedef struct phx_model_config {
  int32_t emb_size;        /* D; the embedding table width equals D */
  int32_t num_layers;
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t key_size;        /* head dim: 32, 64 or 128 */
  int32_t ffn_size;
  int32_t history_len;     /* S */
  int32_t num_candidates;  /* C (0 for a user-tower engine) */
  int32_t max_batch;       /* largest request batch a call may carry */
  int32_t num_actions;     /* V discrete heads */
  int32_t num_continuous;  /* continuous heads (slot 0 = dwell time) */
  int32_t num_action_types;
  int32_t num_surfaces;
  int32_t rotary;          /* 1 = RoPE on q,k (layers.py:259-264) */
  int32_t qk_norm;         /* 1 = joint all-heads RMS norm of q and k (normalization.py:46-48) */
  int32_t primer_norm;     /* 1 = post-attn / post-ffn norms (transformer.py:531-533) */
  int32_t cap_method;      /* 0 none, 1 soft_sign, 2 tanh (pallas/ranker_attention_v2.py:118-124) */
  float attn_logit_cap;
  float final_logit_cap;   /* recsys_model.py:4838-4839; <= 0 disables */
  float rms_eps;
  float rope_base;
  float dwell_norm_scale;  /* recsys_model.py:712-733 */
  phx_hash_family user, item, author, ip; /* unified table regions, recsys_embedding.py:234-248 */
  /* Row sharding of the unified table over `table_world` engines (one per GPU) in contiguous ranges, the
   * ownership rule of the reference's row-sharded embedding (phoenix/xrex/cuda/row_emb/src/row_emb_kernel.hpp:
   * 19-25: owner = row / rows_per_rank).  This engine allocates shard `table_rank` only and reads the other
   * shards through peer mappings (phx_table_attach_peer*).  0 or 1 = not sharded. */
  int32_t table_world;
  int32_t table_rank;
  /* The last `num_candidate_only_layers` layers update the candidate rows only: the history rows keep the values
   * they had on entering that tail, every tail layer projects its keys / values from those frozen rows, and QKV
   * (queries), out-projection and FFN run over the candidate rows alone (phoenix/xrex/models/transformer.py:
   * 789-871, 908-941; layers.py:589-725; production value 2, configs/xrecsys.py:554-555).  0 = every layer
   * updates every row.  Applies to the ranking forward; the user tower has no candidates. */
  int32_t num_candidate_only_layers;
  /* 1 = full-precision path: every activation in fp32 (weights the same bf16-representable values), plain SIMT
   * kernels; the precision of the reference's CPU-runnable fp32 model, for parity runs (within 1e-5 of the fp32
   * model), not for throughput.  0 = bf16 activations with fp32 accumulation on the tcgen05 kernels. */
  int32_t compute_fp32;
  /* How the gathered rows of a token are combined.  0: summed in fp32 in slot order, one rounding (the benchmark's
   * restatement).  1: laid side by side and multiplied by a projection matrix, the reference's own form
   * (block_history_reduce / block_candidate_reduce, recsys_model.py:2163-2365: concat(post rows, author rows
   * [, action row, surface row]) @ proj_mat): parameters "proj_hist" [(2H+2)*emb_size, emb_size] and "proj_cand"
   * [2H*emb_size, emb_size]. */
  int32_t token_project;
  /* 1 = ragged batches are packed: phx_rank_forward (host buffers) counts each request's leading non-padding history
   * slots and candidates and the forward runs over those rows only, back to back (the reference serves ragged users
   * through sequence packing, phoenix/xrex/data/sequence_packing.py:317; here the packing is by rows, requests stay
   * independent).  Requests must be front-filled (padding only behind the valid slots); a batch that is not is run
   * over all its slots.  Outputs of padded candidate slots are zero.  phx_rank_forward and phx_rank_submit pack (they
   * see the ids on the host); the device-pointer entry points run over all slots. */
  int32_t pack_ragged;
  /* 1 = the history actions of a position are a SET: hist_actions holds a bit mask (bit v = action v, v <
   * num_action_types <= 32; the reference's bool[B,S,V] buffer packed), and "action_table" is one [1, emb_size] vector
   * cut into num_action_types chunks, chunk v signed by 2 a_v - 1, the row zero where no action is set
   * (multi_hot_to_embeddings, recsys_model.py:3259-3314).  emb_size / num_action_types must be a multiple of 8.
   * 0 = one action id per position looked up in a [num_action_types + 1, emb_size] table. */
  int32_t action_multi_hot;
  /* The remaining fields describe the reference's batch-prep buffers beyond posts and authors
   * (xai-recsys-engine/src/python.rs:1394-1404); they are served by phx_rank_forward_prep* only.
   * user_prefix: 1 = every request starts with one user token in front of its history (block_user_reduce,
   * recsys_model.py:1889-1927): the rows of user_hashes [B, user.num_hashes] side by side times "proj_user"
   * [user.num_hashes * emb_size, emb_size] (token_project = 1; summed in slot order with token_project = 0), plus
   * the sum of the rows of user_ip_hashes [B, ip.num_hashes] when ip.num_hashes > 0.  The token is valid when
   * user_hashes[b, 0] != 0, sits at position 0 and is attended like a history row (recsys_model.py:4720-4724,
   * 2493-2505); history position s moves to s + 1 and the candidates to history_len + 1. */
  int32_t user_prefix;
  /* 1 = candidate tokens take the row candidate_product_surfaces[b, c] of "surface_table" as one more slot behind
   * the author rows (block_candidate_reduce, recsys_model.py:2278-2365); "proj_cand" is then
   * [(2H+1) * emb_size, emb_size]. */
  int32_t cand_surface;
  /* Continuous history actions (block_history_reduce, recsys_model.py:2249-2271; project_continuous_value_to_embedding,
   * 1850-1886; normalize_continuous_value, 1756-1765): for i < num_hist_continuous the value
   * history_continuous_actions[b, s, hist_cont_index[i]] is clipped to [0, hist_cont_norm_scale[i]], normalised
   * (log1p(v) / log1p(scale) when hist_cont_use_log[i], else v / scale), sent through gelu(v * proj1) @ proj2 with
   * parameters "hist_cont<i>.proj1" [1, hist_cont_hidden] and "hist_cont<i>.proj2" [hist_cont_hidden, emb_size], and
   * the result is added to the history token, one rounding to the activation type per addend.  hist_cont_hidden is
   * 32 or 64 (the reference's 64). */
  int32_t num_hist_continuous;
  int32_t hist_cont_hidden;
  int32_t hist_cont_index[PHX_MAX_HIST_CONT];
  int32_t hist_cont_use_log[PHX_MAX_HIST_CONT];
  float hist_cont_norm_scale[PHX_MAX_HIST_CONT];
  int32_t _pad3;
} phx_model_config;

/* Weighted blend in term-list form: xai-value-model/scoring.rs:67-73, 112-120, 282-291.
 * score = offset_score(sum_i value[src[i]] * weight[i]) summed left to right in f64, where
 * value[j] = exp(log_prob[j]) for j < num_actions, continuous[j - num_actions] otherwise. */
typedef struct phx_blend_spec {
  int32_t num_terms;
  int32_t src[PHX_MAX_BLEND_TERMS];
  double weight[PHX_MAX_BLEND_TERMS];
  double total_sum;    /* ValueModelWeights::offset_total_sum, xai-value-model/weights.rs:107-113 */
  double negative_sum; /* ValueModelWeights::offset_negative_sum, weights.rs:99-105 */
} phx_blend_spec;

/* One batch of ranking requests, the buffers the reference's batch-prep hands the model
 * (xai-recsys-engine/src/python.rs:1394-1440) with raw int64 ids in place of pre-hashed rows:
 * hashing runs on the device.  id 0 = padding; history is front-filled. */
typedef struct phx_rank_batch {
  int32_t batch;
  int32_t _pad;
  const int64_t* hist_post_ids;   /* [B,S] */
  const int64_t* hist_author_ids; /* [B,S] */
  const int32_t* hist_actions;    /* [B,S] 1..num_action_types, 0 = none */
  const int32_t* hist_surfaces;   /* [B,S] 1..num_surfaces, 0 = none */
  const int64_t* cand_post_ids;   /* [B,C] */
  const int64_t* cand_author_ids; /* [B,C] */
} phx_rank_batch;

/* The same batch as the reference's batch-prep fills it (xai-recsys-engine/src/python.rs:1394-1440:
 * history_post_hashes / history_auth_hashes i32[B,S,H], candidate_post_hashes / candidate_auth_hashes i32[B,C,H]):
 * rows of the unified table, already hashed and offset on the host (recsys_embedding.py:282-331), 0 = padding,
 * rows outside the table read row 0 (emb_table.rs:134-137).  Actions / surfaces as in phx_rank_batch. */
typedef struct phx_rank_batch_hashed {
  int32_t batch;
  int32_t _pad;
  const int32_t* hist_post_hashes;   /* [B,S,H] */
  const int32_t* hist_author_hashes; /* [B,S,H] */
  const int32_t* hist_actions;       /* [B,S] */
  const int32_t* hist_surfaces;      /* [B,S] */
  const int32_t* cand_post_hashes;   /* [B,C,H] */
  const int32_t* cand_author_hashes; /* [B,C,H] */
} phx_rank_batch_hashed;

/* The mandatory buffers of the reference's batch-prep, as it fills them and under its names
 * (xai-recsys-engine/src/python.rs:1394-1404).  Hash arrays hold rows of the unified table (0 = padding).
 * history_actions is the bool [B,S,V] array itself, one byte per flag, V = num_action_types (the engine needs
 * action_multi_hot = 1).  Which buffers are read follows the configuration: user_hashes / user_ip_hashes with
 * user_prefix, candidate_product_surfaces with cand_surface, history_continuous_actions with
 * num_hist_continuous > 0; the others may be NULL. */
#define PHX_PREP_CONTINUOUS 8   /* columns of history_continuous_actions (xai-recsys/src/util.rs) */
typedef struct phx_rank_batch_prep {
  int32_t batch;
  int32_t _pad;
  const int32_t* user_hashes;                /* [B, user.num_hashes] */
  const int32_t* user_ip_hashes;             /* [B, ip.num_hashes] */
  const int32_t* history_post_hashes;        /* [B,S,H] */
  const int32_t* history_auth_hashes;        /* [B,S,H] */
  const int32_t* history_product_surfaces;   /* [B,S] */
  const uint8_t* history_actions;            /* bool [B,S,V] */
  const float* history_continuous_actions;   /* [B,S,PHX_PREP_CONTINUOUS] */
  const int32_t* candidate_post_hashes;      /* [B,C,H] */
  const int32_t* candidate_auth_hashes;      /* [B,C,H] */
  const int32_t* candidate_product_surfaces; /* [B,C] */
} phx_rank_batch_prep;

/* Outputs of a ranking call, the arguments of the reference's reply
 * (xai-recsys-engine/src/python.rs:390-396) plus the blended score.  Any pointer may be NULL. */
typedef struct phx_rank_out {
  float* log_probs;   /* [B,C,V]  ln sigmoid(logit), f32 (model_runner.py:4474) */
  float* continuous;  /* [B,C,NC] */
  double* scores;     /* [B,C]    weighted score (scoring.rs:67-73) */
} phx_rank_out;

typedef struct phx_engine phx_engine;

/* ---- lifecycle ------------------------------------------------------------------------------ */

/* Replaces model construction + executable build of the model runner
 * (model_runner.py:2578-2652, 4303-4342).  Allocates weights, the unified embedding table and all
 * work space for `max_batch` on `device`. */
phx_status phx_engine_create(const phx_model_config* cfg, int32_t device, phx_engine** out);
void phx_engine_destroy(phx_engine* e);
/* Text of the last error on this engine (never NULL).  Replaces the string errors of the plugin
 * seam (candidate-pipeline/scorer.rs:29-44). */
const char* phx_last_error(const phx_engine* e);
/* Library-level message for failures before an engine exists. */
const char* phx_global_error(void);

/* ---- parameters ------------------------------------------------------------------------------ */

/* Load one dense parameter from host memory as float32 [rows, cols] row-major in the reference's
 * (in, out) orientation (linear_layer.py:66-82); values are rounded to bf16 on load, as the
 * reference reads parameters (model_utils.py:160-169).  Names: "action_table", "surface_table",
 * "final_norm", "unembed", "cont_unembed", "layer<i>.{pre_attn_norm,w_qkv,q_norm,k_norm,w_out,
 * post_attn_norm,pre_ffn_norm,w_up,w_down,post_ffn_norm}"; with token_project "proj_hist", "proj_cand" (and
 * "proj_user" with user_prefix); "hist_cont<i>.{proj1,proj2}" with continuous history actions. */
phx_status phx_load_param(phx_engine* e, const char* name, const float* host, int64_t rows, int64_t cols);
/* Upload rows [row0, row0+nrows) of the unified embedding table (bf16 bit patterns).  Replaces
 * the engine's table load (xai-recsys-engine/src/emb_table.rs). */
phx_status phx_table_upload(phx_engine* e, int64_t row0, int64_t nrows, const uint16_t* host_bf16);
/* Fill the whole table on the device with the deterministic synthetic content used by the
 * benchmark (a pure function of row, column, seed); cf. the reference's lazy random fill of
 * touched rows, phoenix/xrex/inference/h2d.py:418-445. */
phx_status phx_table_fill_synthetic(phx_engine* e, uint32_t seed, float amp);
phx_status phx_set_blend(phx_engine* e, const phx_blend_spec* spec);

/* Row-sharded tables.  Replaces the reference's id / row exchange (phoenix/xrex/cuda/row_emb/src/row_emb_comm.cc:
 * 655-743: all-to-all of ids, owner-side gather, all-to-all of rows) by direct loads from the owner's shard over
 * NVLink inside the gather kernel: each engine exports its shard once, every other engine maps it, and the
 * hash -> gather -> fixed-order sum kernel dereferences whichever shard owns a row.  The sum order is by hash
 * slot and does not depend on the number of shards, so results are bit-identical to the unsharded table. */
#define PHX_IPC_HANDLE_BYTES 64
/* Export this engine's shard for another process (a CUDA IPC memory handle). */
phx_status phx_table_ipc_handle(phx_engine* e, uint8_t out[PHX_IPC_HANDLE_BYTES]);
/* Map shard `rank` exported by another process. */
phx_status phx_table_attach_peer(phx_engine* e, int32_t rank, const uint8_t handle[PHX_IPC_HANDLE_BYTES]);
/* Same-process variants: the device pointer of this engine's shard / attach a shard by pointer (engines of one
 * process, devices with peer access enabled or the same device). */
phx_status phx_table_local_ptr(phx_engine* e, void** out);
phx_status phx_table_attach_peer_ptr(phx_engine* e, int32_t rank, const void* shard_dev);

/* ---- ranking ---------------------------------------------------------------------------------- */

/* Ranking forward with HOST buffers: copies ids in, runs hash -> gather-sum -> transformer ->
 * heads -> blend, copies results out, returns when they are readable.  Replaces
 * RankingModelRunner.gather_embeddings_and_forward + reply (model_runner.py:4141-4222). */
phx_status phx_rank_forward(phx_engine* e, const phx_rank_batch* batch_host, const phx_rank_out* out_host);
/* Row-sharded table with the rows exchanged in bulk between the two halves of a forward (parallel.ShardedRanker):
 * phx_rank_rows_device writes the unified-table row of every token slot (int32 [B, S+C, 2*num_hashes]: post hashes,
 * then author hashes) on `stream` (a cudaStream_t; NULL = the engine's stream) and stops; after the exchange (phx_shard_*), phx_rank_forward_rows_device runs the forward
 * taking slot j of token t from landing_dev[pos_dev[t * 2*num_hashes + j]] (bf16 rows of emb_size) instead of the
 * table.  Same results as phx_rank_forward_device on an unsharded table, bit for bit.  The reference does the same
 * split around its row_emb exchange (row_emb_comm.cc:655-743). */
phx_status phx_rank_rows_device(phx_engine* e, const phx_rank_batch* batch_dev, int32_t* rows_dev, void* stream);
phx_status phx_rank_forward_rows_device(phx_engine* e, const phx_rank_batch* batch_dev, const uint16_t* landing_dev,
                                        const int32_t* pos_dev, const phx_rank_out* out_dev);
/* Two-deep pipeline of host-buffer requests: phx_rank_submit copies the inputs into the slot's pinned block and
 * enqueues H2D copy, forward and D2H copies (the copies on their own stream: they overlap the forward of the other
 * slot); phx_rank_collect waits for the slot's results and copies them out.  Same semantics as phx_rank_forward per
 * request; a slot must be collected before it is submitted again (PHX_E_STATE otherwise).  A serving loop that keeps
 * both slots in flight hides the host-side copies behind the forward — the reference runner's async dispatch /
 * reply split (model_runner.py:4141-4222). */
phx_status phx_rank_submit(phx_engine* e, const phx_rank_batch* batch_host, int32_t slot);
phx_status phx_rank_collect(phx_engine* e, int32_t slot, const phx_rank_out* out_host);
/* Same with DEVICE buffers, asynchronous on the engine's stream (call phx_sync to wait). */
phx_status phx_rank_forward_device(phx_engine* e, const phx_rank_batch* batch_dev, const phx_rank_out* out_dev);
/* The ranking forward from pre-hashed rows (phx_rank_batch_hashed): the drop-in for a host that keeps the reference's
 * own batch-prep (compute_batch_inputs_rust_quick, model_runner.py:3072-3077) and hands over its buffers unchanged.
 * Device buffers, asynchronous on the engine's stream; results identical to phx_rank_forward_device on the ids the
 * rows were hashed from.  phx_rank_forward_hashed is the same with HOST buffers, blocking like phx_rank_forward. */
phx_status phx_rank_forward_hashed_device(phx_engine* e, const phx_rank_batch_hashed* batch_dev, const phx_rank_out* out_dev);
phx_status phx_rank_forward_hashed(phx_engine* e, const phx_rank_batch_hashed* batch_host, const phx_rank_out* out_host);
/* The ranking forward from the reference's batch-prep buffers as they are (phx_rank_batch_prep): what
 * ModelRunner.predict receives from RankingBatchPrep (xai-recsys-engine/src/python.rs:1394-1440,
 * phoenix/xrex/inference/model_runner.py:4440-4479).  _device: device pointers, asynchronous on the engine's stream.
 * The host form stages the buffers through pinned memory, runs and waits.  The id entry points (phx_rank_forward and
 * the rest) refuse an engine configured with user_prefix, cand_surface or continuous history actions: they carry
 * none of those buffers. */
phx_status phx_rank_forward_prep_device(phx_engine* e, const phx_rank_batch_prep* batch_dev, const phx_rank_out* out_dev);
phx_status phx_rank_forward_prep(phx_engine* e, const phx_rank_batch_prep* batch_host, const phx_rank_out* out_host);
/* Packed rows for callers whose batches already sit on the device (pack_ragged engines).  phx_plan_ragged is the
 * host-side count phx_rank_forward does itself: for B requests of S history and C candidate slots (int64 post ids,
 * 0 = padding) it writes the exclusive prefix sums hist_off / cand_off (B + 1 entries each) of every request's leading
 * non-padding slots - at least one history row per request, all slots for every request when some request has
 * padding in front of a valid slot; it touches no GPU.  phx_rank_forward_packed_device runs the forward over those rows:
 * the two offset arrays in DEVICE memory, hist_rows = hist_off[B], cand_rows = cand_off[B]; outputs keep their [B, C]
 * shape, padded slots read zero.  The role of the reference's packed serving layout (sequence_packing.py:317). */
phx_status phx_plan_ragged(const int64_t* hist_post_ids, const int64_t* cand_post_ids, int32_t B, int32_t S, int32_t C,
                           int32_t* hist_off, int32_t* cand_off);
phx_status phx_rank_forward_packed_device(phx_engine* e, const phx_rank_batch* batch_dev, const int32_t* hist_off_dev,
                                          const int32_t* cand_off_dev, int64_t hist_rows, int64_t cand_rows,
                                          const phx_rank_out* out_dev);
/* Build the tokens (hash -> gather-sum) of the batch that the NEXT phx_rank_forward_device call will carry, on a
 * side stream, so that the gather - which waits on other GPUs' memory when the table is row-sharded - overlaps the
 * forward that is already enqueued.  Call order per step: forward(batch i), then prefetch(batch i+1).  The next
 * forward whose batch descriptor is identical adopts the prefetched tokens; any other batch discards them.
 * Replaces the overlap the reference gets from its embedding side stream
 * (phoenix/xrex/cuda/row_emb/src/row_emb_comm.hpp:228). */
phx_status phx_rank_prefetch_device(phx_engine* e, const phx_rank_batch* batch_dev);
phx_status phx_sync(phx_engine* e);
/* Failure detection on the device.  Every wait inside the tcgen05 kernels (on an mbarrier that a TMA copy, an MMA
 * commit or another warp role signals) is bounded: when the limit passes, the waiting thread raises the engine's error
 * flag, every role drains, the kernel returns, and the next blocking call (phx_rank_forward, phx_rank_collect, phx_sync)
 * reports PHX_E_TIMEOUT once and clears the flag; the context stays usable.  phx_set_wait_limit_us sets the limit
 * (microseconds; 0 = the default of 2 s; synchronises the engine's stream).  phx_wait_selftest launches a one-thread
 * kernel that waits on a barrier nothing signals and returns what phx_sync returns after it: PHX_E_TIMEOUT after
 * about one limit when the mechanism works.  The reference leaves hangs to its serving shell (per-request deadlines,
 * xai-recsys-engine/src/request_queue.rs:10-27); a kernel of its own that waits for ever holds the GPU. */
phx_status phx_set_wait_limit_us(phx_engine* e, uint32_t microseconds);
phx_status phx_wait_selftest(phx_engine* e);
/* Which kernel variants the library's launches took, counted over the life of the process: out[i] for i < n receives the
 * count of variant i, the return value is the number of variants; phx_dispatch_name(i) names them ("attn.strip",
 * "attn.stream", "attn.tcgen05", "attn.resident", "gemm.pair256", "gemm.pair128", "gemm.cta256", "gemm.cta128",
 * "gemm.simt", "scan.tcgen05", "scan.mma", "topk.exact").  A forward replayed from its CUDA graph counts nothing.  Lets a
 * test or a monitor assert that a workload runs on the kernels meant for it.  The reference's counterpart is its
 * attention-implementation switch being logged at start-up (phoenix/xrex/models/recsys_attention.py:18-242). */
int32_t phx_dispatch_counts(int64_t* out, int32_t n);
const char* phx_dispatch_name(int32_t kind);
/* Time of the last phx_rank_forward_device / phx_user_tower_device call on the engine's stream,
 * measured with CUDA events (milliseconds). */
phx_status phx_last_device_ms(phx_engine* e, float* ms);
/* Device-side timing on the engine's stream: phx_mark records event `slot` (0..7) behind the work
 * queued so far, phx_elapsed_ms waits for `to_slot` and returns the time between two marks, phx_mark_wait
 * blocks the host until the work in front of a mark is done (a mark never recorded is done).  Replaces
 * the reference's per-step latency metrics (model_runner.py:3089-3092, 4176-4179). */
phx_status phx_mark(phx_engine* e, int32_t slot);
phx_status phx_mark_wait(phx_engine* e, int32_t slot);
phx_status phx_elapsed_ms(phx_engine* e, int32_t from_slot, int32_t to_slot, float* ms);
/* Per-kernel-class timing of the last forward (CUDA events around every launch while enabled).
 * Classes: 0 token build (hash + gather-sum), 1 RMSNorm, 2 GEMM, 3 qk-norm/RoPE, 4 attention,
 * 5 heads + blend.  Arrays of 6.  Replaces the reference's profiler annotations
 * (model_runner.py:3068-3071, 4157-4160). */
phx_status phx_profile_enable(phx_engine* e, int32_t on);
phx_status phx_profile_read(phx_engine* e, float* ms_by_class, int32_t* launches_by_class);
/* Number of kernel launches the last forward issued. */
phx_status phx_last_launch_count(phx_engine* e, int32_t* n);

/* Debug / parity taps after a forward (device -> host copies of internal buffers):
 * "hashes" int32 [B,T,2H] (post hashes then author hashes per token), "tokens" bf16 bits [B,T,D]
 * (the gather-sum output before scaling), "hidden" bf16 bits [B,T,D] (trunk output). */
phx_status phx_debug_read(phx_engine* e, const char* what, void* host, size_t nbytes);

/* ---- row-sharded table, exchange by all-to-all ------------------------------------------------------------------
 * The device-side steps of the reference's id / row exchange (phoenix/xrex/cuda/row_emb/src/row_emb_comm.cc:655-743:
 * all-to-all of ids, owner-side gather, all-to-all of rows; combine by sum as recsys_embedding.py:282-331).  The two
 * collectives themselves are issued by the host side (NCCL, `parallel.ShardedGatherSum`).  All pointers are device
 * pointers, `stream` is a cudaStream_t (null = default stream); nothing is allocated; errors: phx_global_error().
 *
 * phx_shard_bucket: rows_dev int32 [n_req] unified-table rows (phx_hash_ids_device) -> counts_dev int32 [world]
 * requests per owning rank (owner = row / rows_per_shard), send_rows_dev int32 [n_req] the owner-local row numbers
 * grouped by owner, pos_dev int32 [n_req] the slot of request i in that grouped order; cursor_dev int32 [world] is
 * scratch (on return: the end of each bucket). */
phx_status phx_shard_bucket(const int32_t* rows_dev, int64_t n_req, int64_t rows_per_shard, int32_t world, int32_t* counts_dev,
                            int32_t* cursor_dev, int32_t* send_rows_dev, int32_t* pos_dev, void* stream);
/* Distinct rows of a request list (ids repeat under a skewed distribution; only distinct rows need to cross the link):
 * table_dev uint64 [table_slots] is scratch (a power of two >= 2 * n_req), slot_dev int32 [n_req] and urows_dev int32
 * [up to n_req] outputs, *nu_dev the number of distinct rows.  urows_dev then goes through phx_shard_bucket (giving
 * upos), and phx_shard_dedup_expand turns that into pos_dev int32 [n_req] for phx_shard_sum_rows.  The reference
 * deduplicates before its exchange as well (the slot_unique / owner_unique workspaces, row_emb_comm.cc:122-136). */
phx_status phx_shard_dedup(const int32_t* rows_dev, int64_t n_req, uint64_t* table_dev, int64_t table_slots, int32_t* slot_dev,
                           int32_t* urows_dev, int32_t* nu_dev, void* stream);
phx_status phx_shard_dedup_expand(const int32_t* slot_dev, const uint64_t* table_dev, const int32_t* upos_dev, int64_t n_req,
                                  int32_t* pos_dev, void* stream);
/* Owner side: out_dev bf16 [m, width] = shard rows local_rows_dev[0..m) (out of range -> row 0, emb_table.rs:124-140). */
phx_status phx_shard_gather_rows(const uint16_t* shard_dev, int64_t shard_rows, const int32_t* local_rows_dev, int64_t m,
                                 int32_t width, uint16_t* out_dev, void* stream);
/* Requester side: out_dev bf16 [n, width], row i = bf16(sum over h of rows_dev[pos_dev[i*num_hashes + h]]) in fp32, in
 * hash-slot order: bit-identical to phx_gather_sum_device on the unsharded table. */
phx_status phx_shard_sum_rows(const uint16_t* rows_dev, const int32_t* pos_dev, int64_t n, int32_t num_hashes, int32_t width,
                              uint16_t* out_dev, void* stream);

/* Owner-side gather with the row transfer folded in (one kernel instead of gather + all-to-all of rows): request j
 * (of m = seg_dev[world]) belongs to requester r with seg_dev[r] <= j < seg_dev[r+1] (int64 [world+1]); its row is
 * stored at row j - seg_dev[r] of dest_dev[r] (uint64 [world]: device addresses, local memory or a peer mapping opened
 * with phx_ipc_open), i.e. straight into the bucket that requester reserved for this owner in its landing buffer.  The
 * host side orders the ranks around it (a collective before the landing buffers are rewritten and after the stores).
 * No counterpart as a single call in the reference: row_emb_comm.cc:655-743 gathers, then runs the collective. */
phx_status phx_shard_gather_push(const uint16_t* shard_dev, int64_t shard_rows, const int32_t* local_rows_dev, int64_t m,
                                 const int64_t* seg_dev, const uint64_t* dest_dev, int32_t world, int32_t width, void* stream);
/* One asynchronous device-to-device copy on `stream`; dst / src may be local memory or a peer mapping (the copy engines
 * move a requester's bucket of gathered rows in one piece). */
phx_status phx_copy_async(void* dst, const void* src, uint64_t bytes, void* stream);
/* Device memory that other processes of the node can map: allocate + export / map / unmap / free.  Stand in for the
 * reference's communicator-owned exchange buffers (row_emb_comm.cc:301-336). */
phx_status phx_ipc_alloc(int32_t device, uint64_t bytes, void** ptr_out, uint8_t handle_out[PHX_IPC_HANDLE_BYTES]);
phx_status phx_ipc_open(int32_t device, const uint8_t handle[PHX_IPC_HANDLE_BYTES], void** ptr_out);
phx_status phx_ipc_close(void* ptr);
phx_status phx_ipc_free(void* ptr);

/* ---- stand-alone operators (micro-benchmarks and parity tests of single kernels) ------------- */

/* Multi-hash id -> unified-table rows; `family`: 0 user, 1 item, 2 author, 3 ip.
 * out_dev int32 [n, num_hashes].  recsys_embedding.py:154-172, 282-331. */
phx_status phx_hash_ids_device(phx_engine* e, int32_t family, const int64_t* ids_dev, int64_t n, int32_t* out_dev);
/* Hash + gather + fixed-order fp32 sum -> bf16 [n, D]; the benchmark's gather-sum workload.
 * Replaces embedding_gather (emb_table.rs:330-398) + the combine. */
phx_status phx_gather_sum_device(phx_engine* e, int32_t family, const int64_t* ids_dev, int64_t n, uint16_t* out_dev);
/* Candidate-isolated attention on caller tensors: q,k,v,out bf16 [B,T,H,dh] (Hkv heads for k,v),
 * seg int32 [B,T] (1 history, -1 candidate, 0 padding), keys considered = [0,hist_len).
 * Replaces the ranker attention kernels (phoenix/xrex/models/recsys_attention.py:18-242). */
phx_status phx_ranker_attention_device(int32_t device, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                       const int32_t* seg, uint16_t* out, int32_t B, int32_t T, int32_t Hq,
                                       int32_t Hkv, int32_t dh, int32_t hist_len, float sm_scale, float cap,
                                       int32_t cap_method, float* device_ms);
/* C[M,N] = epilogue(A[M,K] @ W) on the engine's GEMM kernel; Wt is [N,K] bf16 (K-major).
 * epilogue: 0 store, 1 add residual R[M,N] (bf16), 2 GELU-tanh.  impl: 0 tcgen05 (CTA pairs sharing 256-row
 * tiles unless PHX_GEMM=cta1), 1 SIMT reference, 2 tcgen05 with one CTA per 128-row tile.
 * Replaces the Linear layers (linear_layer.py:52-91). */
phx_status phx_gemm_device(int32_t device, const uint16_t* A, const uint16_t* Wt, const uint16_t* R, uint16_t* C,
                           int64_t M, int32_t N, int32_t K, int32_t epilogue, int32_t impl, float* device_ms);

/* ---- retrieval -------------------------------------------------------------------------------- */

/* User tower: history tokens -> transformer -> masked mean pool -> L2 normalise -> f32 [B,D]
 * (recsys_two_tower_model.py:2065-2203).  Uses hist_* of the batch only. */
phx_status phx_user_tower_device(phx_engine* e, const phx_rank_batch* batch_dev, float* users_dev);

typedef struct phx_corpus phx_corpus;
/* A corpus shard of `rows` x `dim` bf16 rows on `device`; global row id = row_offset + local row
 * (recsys_two_tower_model.py:216).  max_queries / max_k size the work space. */
phx_status phx_corpus_create(int32_t device, int64_t rows, int32_t dim, int64_t row_offset, int32_t max_queries,
                             int32_t max_k, phx_corpus** out);
void phx_corpus_destroy(phx_corpus* c);
phx_status phx_corpus_upload(phx_corpus* c, int64_t row0, int64_t nrows, const uint16_t* host_bf16);
/* Copy shard rows [row0, row0 + nrows) (bf16 bit patterns) into a device buffer of the shard's device; returns when
 * the copy is done.  What an index refresh reads back to verify an upload (the reference rebuilds its post table from
 * phoenix-rankall/ snapshots). */
phx_status phx_corpus_read_device(phx_corpus* c, int64_t row0, int64_t nrows, uint16_t* out_dev);
/* Synthetic L2-normalised rows, a pure function of (global row, seed). */
phx_status phx_corpus_fill_synthetic(phx_corpus* c, uint32_t seed);
/* int8 form of the shard (the reference's post_q8 / post_scales table, recsys_two_tower_model.py:2518-2533): rows as
 * int8 [rows, dim] with one float scale per row; a call scores
 *   bf16((float(int32 dot of the int8 query with the int8 row) * query_scale) * row_scale)
 * where the query is quantised per call: query_scale = max(max|u| / 127, 1e-12), q = clip(round_half_even(u /
 * query_scale), -127, 127) (2523-2526).  Integer dot products are exact, so scores and ids are bit-exact against the
 * reference arithmetic.  dim must be a multiple of 32.  phx_corpus_upload_int8 takes the table as the host has it;
 * phx_corpus_quantize_int8 derives it on the device from the resident bf16 rows with the same rule as the queries
 * (benchmarks, tests).  phx_corpus_set_int8(1) makes every later top-k of the shard (windows, masks, keys, exact
 * passes, phx_retrieve_topk) score with the int8 form; it reads half the bytes per row. */
phx_status phx_corpus_upload_int8(phx_corpus* c, int64_t row0, int64_t nrows, const int8_t* host_q8, const float* host_scales);
phx_status phx_corpus_quantize_int8(phx_corpus* c);
phx_status phx_corpus_set_int8(phx_corpus* c, int32_t on);
phx_status phx_corpus_read_int8_device(phx_corpus* c, int64_t row0, int64_t nrows, int8_t* q8_dev, float* scales_dev);
/* Exhaustive dot-product top-k of this shard: users f32 [B,dim] (rounded to bf16 as the reference
 * does), scores bf16-rounded f32 [B,k], ids int64 [B,k] global rows, ordered by (score desc,
 * id asc).  Replaces compute_top_k + top_k_by_key (recsys_two_tower_model.py:2455-2516,
 * cuda/top_k_by_key/__init__.py:56-94).  Asynchronous on the corpus' stream. */
phx_status phx_corpus_topk_device(phx_corpus* c, const float* users_dev, int32_t B, int32_t k, float* scores_dev,
                                  int64_t* ids_dev);
/* The per-shard list in the form it travels in before a merge: one 64-bit key per entry, (order-preserving image of
 * the f32 score) << 32 | ~(row as u32), sorted descending, 0 = empty slot - 8 bytes per entry in ONE all-gather instead
 * of a score and an id array in two (recsys_two_tower_model.py:215-220 gathers both).  phx_topk_merge_keys_device
 * merges [P,B,k] such lists into scores f32 [B,k] and rows int64 [B,k] by (score desc, row asc).  Rows must fit 32
 * bits, as everywhere in this library. */
phx_status phx_corpus_topk_keys_device(phx_corpus* c, const float* users_dev, int32_t B, int32_t k, uint64_t* keys_dev);
phx_status phx_topk_merge_keys_device(phx_corpus* c, const uint64_t* keys_dev, int32_t P, int32_t B, int32_t k,
                                      float* out_scores_dev, int64_t* out_ids_dev);
/* Enqueue the shard's later work on `stream` (a cudaStream_t of the shard's device; NULL is the default stream)
 * instead of its own stream, so that it orders with the caller's other work - the collective between top-k and merge -
 * without host synchronisation; use_own != 0 returns to the shard's own stream.  The reference's ops run on the framework's stream the same way
 * (top_k_by_key_ffi.cc:15-26). */
phx_status phx_corpus_set_stream(phx_corpus* c, void* stream, int32_t use_own);
/* Per-row eligibility of the shard (the reference's per-post masks ahead of the top-k: dataset type mask and
 * eligibility mask, recsys_two_tower_model.py:2486-2493, 2690-2702, where a masked post's score becomes
 * finfo(bf16).min): bit (r & 31) of host_bits[r >> 5] set = shard-local row r may be returned; ceil(rows / 32) words;
 * NULL removes the mask.  Every later top-k call on this shard skips the other rows; when a window holds fewer
 * eligible rows than k, the list is completed with the window's first masked rows at finfo(bfloat16).min in ascending
 * row order, which is what the reference's top-k over the masked scores returns.  Synchronises the shard's stream. */
phx_status phx_corpus_set_mask(phx_corpus* c, const uint32_t* host_bits);
/* The same top-k over rows [row_begin, row_end) of the shard only (shard-local row numbers): the reference's dataset
 * windows, where every retrieval dataset is a contiguous row range of the post table and each gets its own top-k
 * (slice_and_top_k, recsys_two_tower_model.py:2660-2686; ids come back offset by the window's start, as there).
 * k must not exceed the window's rows. */
phx_status phx_corpus_topk_window_device(phx_corpus* c, const float* users_dev, int32_t B, int32_t k, int64_t row_begin,
                                         int64_t row_end, float* scores_dev, int64_t* ids_dev);
/* Merge P per-shard lists laid out [P,B,k] into [B,k] by (score desc, id asc)
 * (strided_dataset_top_k, recsys_two_tower_model.py:215-220).  Ids must be below 2^32; a negative id marks an empty
 * slot (sorted last, returned as score -inf, id -1 when the lists hold fewer than k entries); an entry with a larger
 * id is left out and the next phx_corpus_sync reports PHX_E_ARG. */
phx_status phx_topk_merge_device(phx_corpus* c, const float* scores_dev, const int64_t* ids_dev, int32_t P,
                                 int32_t B, int32_t k, float* out_scores_dev, int64_t* out_ids_dev);
/* The same merge for callers that must not allocate device memory.  (No counterpart in the reference.)
 * Some hosts of this library hand it a stream and buffers but own all device memory themselves: a
 * custom-call handler running inside a compiler-managed step, or a serving process whose memory pool
 * was sized up front and leaves nothing for cudaMalloc, which would also stall the device.  This entry
 * point calls no cudaMalloc / cudaFree and no allocating library routine: its scratch (the 64-bit sort
 * keys and a status word) is a fixed 16 MiB array inside the library image, present on every device
 * that loads the library until the process exits.
 *   - limit: P * B * k <= 2,097,152 keys (e.g. 8 shards x 256 queries x k = 1000); larger merges are
 *     refused with PHX_E_CAPACITY and belong to phx_topk_merge_device;
 *   - the first call on a device looks up the array's device address (once per device, with that
 *     device current); make that first call before any stream capture begins;
 *   - all calls share the one array, which keeps the previous call's contents: the entry point clears
 *     what must start at zero itself, but two calls whose kernels overlap on the GPU (different
 *     streams, no ordering between them) race on it; order them;
 *   - asynchronous on `stream` (a cudaStream_t, NULL = the default stream); inputs and outputs are the
 *     caller's device buffers, laid out as for phx_topk_merge_device;
 *   - ids must be below 2^32 (negative = empty slot): an entry with a larger id is left out of the merge and
 *     bit 2 of the status word is raised.  phx_topk_merge_static_status waits for `stream`, copies that word
 *     to the host (a 4-byte copy, no allocation) and returns it in *status_out: 0 = every entry was merged;
 *   - the calling thread's current device is the same after the call as before it. */
phx_status phx_topk_merge_static(int32_t device, const float* scores_dev, const int64_t* ids_dev, int32_t P,
                                 int32_t B, int32_t k, float* out_scores_dev, int64_t* out_ids_dev, void* stream);
phx_status phx_topk_merge_static_status(int32_t device, void* stream, int32_t* status_out);
/* Wait for the shard's work and report what went wrong in it.  The fast top-k keeps the rows at or above a pivot
 * estimated from a sample of the corpus; when a query's pivot turns out too high (fewer than k rows reach it) or too low
 * (more rows than the survivor buffer holds: long runs of equal scores, clustered rows), the sync does that call again
 * with exact thresholds - bisection on the 64-bit (score, row) key with one counting scan per step - into the same output
 * buffers, so a top-k call followed by a sync always yields the exhaustive answer, as the reference's top_k does
 * (cuda/top_k_by_key/__init__.py:56-94).  The query buffer of the call must still hold the queries.
 * phx_corpus_finish is the same and tells in *reran_out whether the call was done again (a caller that has already
 * passed the first answer on - an all-gather of the lists - then repeats that step).  phx_corpus_set_exact(on) makes
 * every later top-k of the shard take the exact passes straight away (synchronous); phx_corpus_exact_runs counts the
 * calls that took them. */
phx_status phx_corpus_sync(phx_corpus* c);
phx_status phx_corpus_finish(phx_corpus* c, int32_t* reran_out);
phx_status phx_corpus_set_exact(phx_corpus* c, int32_t on);
phx_status phx_corpus_exact_runs(phx_corpus* c, int64_t* n);
phx_status phx_corpus_last_device_ms(phx_corpus* c, float* ms);
const char* phx_corpus_last_error(const phx_corpus* c);

/* ---- multi-GPU: the library's own communicator --------------------------------------------------------------------
 * One process per GPU.  The library owns an NCCL communicator per rank, as the reference's row-sharded embedding does
 * (phoenix/xrex/cuda/row_emb/src/row_emb_comm.cc:283-345: rank 0 makes a unique id, the host ships it to the other
 * ranks, every rank joins), so a host without any ML framework can run the sharded paths: phx_comm_unique_id on rank
 * 0, the id to the other processes by the host's own means, phx_comm_create on every rank (collective).  NCCL is
 * loaded at run time (libnccl.so.2); PHX_E_NCCL reports a missing library or a failed NCCL call, text in
 * phx_comm_last_error.  phx_comm_barrier waits for every rank (collective). */
#define PHX_COMM_ID_BYTES 128
typedef struct phx_comm phx_comm;
phx_status phx_comm_unique_id(uint8_t out[PHX_COMM_ID_BYTES]);
phx_status phx_comm_create(const uint8_t id[PHX_COMM_ID_BYTES], int32_t rank, int32_t world, int32_t device, phx_comm** out);
void phx_comm_destroy(phx_comm* c);   /* collective when the sharded gather was set up: ranks unmap each other's buffers first */
const char* phx_comm_last_error(const phx_comm* c);
phx_status phx_comm_info(const phx_comm* c, int32_t* rank, int32_t* world, int32_t* nccl_version);
phx_status phx_comm_barrier(phx_comm* c, void* stream);

/* Two-tower retrieval over a corpus row-sharded across the ranks, as one call (collective; every rank passes the same
 * queries): this rank's shard is scanned for its top-k, the per-shard lists travel in one NCCL all-gather (one 64-bit
 * key per entry) together with every shard's status word, every rank merges them by (score desc, row asc) into
 * scores_dev f32 [B,k] / ids_dev int64 [B,k] (global rows), and the call returns when the result is ready.  If the
 * sampled pivot missed on any shard, that shard repeats its scan with exact thresholds and all ranks gather and merge
 * again, so the answer is always the exhaustive top-k.  Replaces compute_top_k under shard_map: shard-local top-k,
 * all_gather, top_k (recsys_two_tower_model.py:2455-2516, 193-221).  `stream`: a cudaStream_t of the shard's device the
 * work is ordered on (NULL = default stream). */
phx_status phx_retrieve_topk(phx_comm* comm, phx_corpus* shard, const float* users_dev, int32_t B, int32_t k,
                             float* scores_dev, int64_t* ids_dev, void* stream);

/* Multi-hash gather-sum over the unified table row-sharded across the ranks (engines created with table_world =
 * world, table_rank = rank), exchange done by the library: the reference's lookup sequence (row_emb_comm.cc:655-743,
 * 868-879) - ids hashed to rows, distinct rows grouped by owner, counts exchanged (one all-gather and the call's only
 * host wait), row numbers sent to their owners (NCCL send / recv), owner-side gather, rows back to the requesters (one
 * copy-engine transfer per peer into the requester's landing buffer, mapped over CUDA IPC), fp32 sum in hash-slot
 * order.  Bit-identical to phx_gather_sum_device on the unsharded table.  phx_gather_sharded_setup (collective, once)
 * sizes the work space for max_ids ids per call; recv_factor bounds the rows one rank may be asked for in a call at
 * recv_factor * max_ids * num_hashes (PHX_E_CAPACITY beyond it, as the reference's row_emb_recv_factor).
 * phx_gather_sum_sharded (collective): this rank's ids_dev int64 [n] -> out_dev bf16 [n, emb_size], asynchronous on
 * `stream` after its one host wait.  phx_gather_sharded_phase_ms: device time of the last call's seven phases on this
 * rank (requester prologue, counts exchange with the host wait, row numbers, owner-side gathers, remaining copies, fence,
 * sum). */
phx_status phx_gather_sharded_setup(phx_comm* comm, phx_engine* e, int64_t max_ids, double recv_factor);
phx_status phx_gather_sum_sharded(phx_comm* comm, phx_engine* e, int32_t family, const int64_t* ids_dev, int64_t n,
                                  uint16_t* out_dev, void* stream);
/* The same for ids of several features in one call: ids_dev holds nseg runs back to back, run i = seg_count[i] ids of
 * hash family seg_family[i] (0 user, 1 item, 2 author, 3 ip; every family used must have the engine's item hash count).
 * One exchange serves all runs, so lookups that spread over the table's regions - the reference gathers every
 * feature of a batch in one row_emb call - load every owner alike; a single-family call sends all of its requests
 * to the one or two ranks that hold that region.  out_dev: [sum of seg_count, emb_size] in id order. */
phx_status phx_gather_sum_sharded_multi(phx_comm* comm, phx_engine* e, int32_t nseg, const int32_t* seg_family,
                                        const int64_t* seg_count, const int64_t* ids_dev, uint16_t* out_dev, void* stream);
phx_status phx_gather_sharded_phase_ms(phx_comm* comm, float* ms7);

/* ---- serving shell: request queue and admission control -----------------------------------------------------------
 * The duties of the reference's serving engine between its wire layer and the model runner's dispatch loop
 * (`server.dequeue()`, model_runner.py:3026-3046), host code only.
 *
 * Request queue (xai-recsys-engine/src/request_queue.rs:10-155): producers push (request id, enqueue time, optional
 * deadline) into a bounded channel (PHX_E_CAPACITY when it is full); phx_queue_dequeue moves requests into the batch
 * under construction, hands out at most batch_size request ids in arrival order, and drops - reporting them in
 * dropped_out, the reference's on_stale_drop - every request that has expired on the way: past its deadline, or, without
 * a deadline, older than max_staleness_us (UINT64_MAX = never).  With batch_wait_us > 0 the call waits up to that long
 * for the batch to fill (from an empty start: for one request), polling every millisecond.  Times are microseconds of
 * one monotonic clock the host chooses (phx_now_us gives one); ids_out must hold batch_size entries. */
typedef struct phx_request_queue phx_request_queue;
uint64_t phx_now_us(void);
phx_status phx_queue_create(int32_t batch_size, int32_t channel_size, uint64_t max_staleness_us, uint64_t batch_wait_us,
                            phx_request_queue** out);
void phx_queue_destroy(phx_request_queue* q);
phx_status phx_queue_push(phx_request_queue* q, uint64_t request_id, uint64_t enqueue_time_us, uint64_t deadline_us /* 0 = none */);
phx_status phx_queue_dequeue(phx_request_queue* q, uint64_t now_us, uint64_t* ids_out, int32_t max_out, int32_t* n_out,
                             uint64_t* dropped_out, int32_t max_dropped, int32_t* n_dropped);
phx_status phx_queue_stats(phx_request_queue* q, int32_t* waiting, uint64_t* total_dropped);

/* Admission control (xai-recsys-engine/src/admission.rs:44-227): a request is refused at the door when the predicted
 * time to its answer exceeds what is left of its deadline.  Two estimators: eta_model 0 ("loop") = (batches ahead +
 * pipeline_depth) * service time + post_us, with the service time an EWMA of phx_admission_record_service_us samples;
 * eta_model 1 ("pipeline") = queue wait + pipeline time + post_us, the pipeline time an EWMA of sojourn samples minus
 * their queue wait.  Nothing is refused while the backlog is below one batch, without an estimate, or without a
 * deadline (remaining_us < 0). */
typedef struct phx_admission_config {
  int32_t enabled;
  int32_t eta_model;           /* 0 loop, 1 pipeline */
  uint64_t batch_size, margin_us, post_us, fallback_budget_us, pipeline_depth;
  double ewma_alpha;           /* outside (0, 1]: 0.2 */
} phx_admission_config;
typedef struct phx_admission phx_admission;
phx_status phx_admission_create(const phx_admission_config* cfg, phx_admission** out);
void phx_admission_destroy(phx_admission* a);
phx_status phx_admission_set_enabled(phx_admission* a, int32_t on);
phx_status phx_admission_reset(phx_admission* a);
phx_status phx_admission_record_service_us(phx_admission* a, uint64_t sample_us);
phx_status phx_admission_record_sojourn_us(phx_admission* a, uint64_t sample_us, int64_t admit_backlog);
/* 1 and *eta_us when an estimate exists, else 0; model < 0 = the configured one */
int32_t phx_admission_predicted_eta_us(phx_admission* a, int64_t queue_depth, int32_t model, uint64_t* eta_us);
int32_t phx_admission_should_reject(phx_admission* a, int64_t remaining_us /* < 0 = no deadline */, int64_t queue_depth);
phx_status phx_admission_estimates(phx_admission* a, uint64_t* service_time_us, uint64_t* pipeline_time_us);

/* ---- value model after the heads (xai-value-model/scoring.rs) ---------------------------------- */

/* PhoenixScores fields in declaration order (xai-value-model/phoenix_scores.rs:2-32): favorite, reply, retweet,
 * photo_expand, video_open, click, open_link, profile_click, vqv, share, share_via_dm, share_via_copy_link, dwell,
 * quote, quoted_click, quoted_vqv, follow_author, not_interested, block_author, mute_author, report, not_dwelled,
 * post_unexplored, post_video, grok_analyze, dwell_time, click_dwell_time, home_video_continuation_secs,
 * home_profile_visit_secs. */
#define PHX_VM_FIELDS 29
#define PHX_VM_TERMS 30
#define PHX_VM_MAX_CANDIDATES 4096

/* ValueModelWeights (xai-value-model/weights.rs:8-53) in the form the scoring functions read it. */
typedef struct phx_value_model {
  /* where each PhoenixScores field comes from: column j < num_actions is exp(log_probs[j]) (the wire conversion,
   * home-mixer/candidate_pipeline/performance_tests.rs:516-521), num_actions + j is continuous[j], -1 = None */
  int32_t src[32];
  /* the weight of each of the 30 terms of weighted_terms, in its order (scoring.rs:145-260), before the per-candidate
   * gates: favorite, reply, retweet, photo_expand, video_open, click, open_link, profile_click, vqv, share,
   * share_via_dm, share_via_copy_link, dwell, quote, quoted_click, quoted_vqv, cont_dwell_time,
   * cont_click_dwell_time, video_continuation, user_video_continuation, profile_visit_secs, follow_author,
   * not_interested, block_author, mute_author, report, not_dwelled, post_unexplored, post_video, grok_analyze */
  double w[PHX_VM_TERMS];
  double reply_boost, dwell_boost;                 /* bidirectional_follow_*_weight_boost */
  double author_diversity_decay, author_diversity_floor;
  double not_dwelled_power_exponent, not_dwelled_power_offset, engage_bias;
  double offset_total_sum, offset_negative_sum;    /* weights.rs:99-113 */
  int32_t post_unexplored_include_oon, enable_author_diversity, oon_rescore_in_network_replies_retweets;
  int32_t multiplier_pre_offset, multiplicative, _pad;
} phx_value_model;

/* bits of phx_value_inputs.flags (CandidateScoringInputs, xai-value-model/inputs.rs:3-17) */
#define PHX_VM_IN_NETWORK_KNOWN 1
#define PHX_VM_IN_NETWORK 2
#define PHX_VM_IS_REPLY 4
#define PHX_VM_IS_RETWEET 8
#define PHX_VM_MUTUAL_FOLLOW 16
#define PHX_VM_VQV_ELIGIBLE 32
#define PHX_VM_QUOTED_VQV_ELIGIBLE 64

/* One batch of requests for the value model: DEVICE pointers, per candidate [B,C] unless noted.  Optional arrays may
 * be NULL. */
typedef struct phx_value_inputs {
  int32_t batch, num_candidates, num_actions, num_continuous;
  const float* log_probs;            /* [B,C,V] as phx_rank_out.log_probs */
  const float* continuous;           /* [B,C,NC] */
  const double* weighted;            /* cached weighted_score (phx_rank_out.scores) or NULL: fuse_heads is run */
  const int64_t* author_ids;
  const uint8_t* flags;              /* PHX_VM_* bits; NULL = all zero */
  const double* exploration_bonus;   /* NULL = 0 */
  const int32_t* cold_start_rank;    /* cold_start_lift_to_rank, -1 = None; NULL = none */
  const int32_t* num_valid;          /* [B] candidates of each request (the rest are ignored); NULL = C */
  const double* context;             /* [B,5] effective_oon_weight, oon engagement / dwell_time factors, in-network
                                        engagement / dwell_time factors (a NaN engagement factor = None); NULL =
                                        QueryScoringContext::default() */
} phx_value_inputs;

/* compute_value_scores (xai-value-model/scoring.rs:404-489) for B requests, one thread block per request:
 * fuse_heads with the per-candidate gates, the multiplicative mode and the request's user_video_continuation
 * (scoring.rs:67-280) unless a cached weighted score is given; exploration bonus; cold-start lift; author diversity
 * (rank among the same author's candidates by score, ties in input order); out-of-network weight; class factors.
 * Writes weighted_out / scores_out f64 [B,C] (weighted_out may be NULL) on `stream` (a cudaStream_t, NULL = default
 * stream).  Replaces home-mixer's value-model scorer calling into xai-value-model on the CPU
 * (home-mixer/scorers/value_model.rs). */
phx_status phx_value_scores_device(int32_t device, const phx_value_model* model, const phx_value_inputs* in,
                                   double* weighted_out, double* scores_out, void* stream);

/* ---- diversity rerank behind the value model (vm-ranker/dpp.rs) --------------------------------------------------- */

#define PHX_DPP_MAX_POOL 96
#define PHX_DPP_MAX_CONTEXT 32

/* DppConfig / SlidingWindow (vm-ranker/dpp.rs:14-29). */
typedef struct phx_dpp_config {
  int32_t top_k;               /* picks wanted, <= 96 */
  int32_t max_selected_rank;   /* pool = this many best-scoring candidates, <= 96 */
  int32_t greedy_order;        /* 1 = serve in pick order */
  int32_t window_on;           /* 1 = sliding-window selection instead of the DPP kernel */
  double theta;
  int32_t window_size;         /* INT32_MAX = unbounded */
  int32_t _pad;
  double half_distance, sid_lambda;
} phx_dpp_config;

/* DppInput arrays of a batch of requests, DEVICE pointers (dpp.rs:31-38): embeddings are IEEE half bit patterns, norms
 * as the caller computed them.  The context is the seed (if has_seed: item 0; only the seed is used without a
 * window) followed by the history, most recent first. */
typedef struct phx_dpp_inputs {
  int32_t batch, num_candidates, emb_dim, num_context;
  const double* scores;             /* [B,C] */
  const uint16_t* embeddings;       /* [B,C,E] */
  const double* norms;              /* [B,C] */
  const uint8_t* missing;           /* [B,C] embedding_missing, or NULL */
  const int32_t* l1;                /* [B,C] first-level semantic id, < 0 = none, or NULL */
  const int32_t* num_valid;         /* [B] candidates of each request, or NULL = C */
  const uint16_t* ctx_embeddings;   /* [B,Hc,E] */
  const double* ctx_norms;          /* [B,Hc] */
  const uint8_t* ctx_missing;       /* [B,Hc] or NULL */
  const int32_t* ctx_l1;            /* [B,Hc] or NULL */
  const int32_t* num_context_valid; /* [B] or NULL = Hc */
  int32_t has_seed;
  int32_t _pad;
} phx_dpp_inputs;

/* `rescore` (vm-ranker/dpp.rs:45-215) for B requests, one thread block each: out_index int32 [B, top_k] = the input
 * index of the candidate served at each position (-1 behind the last pick), out_score f64 [B, top_k] = the score shown
 * at that position (the picks' scores in descending order, whatever the serving order), out_count int32 [B].  Equal
 * scores are ordered by input index where the reference's unstable sort leaves the order open; the dot product is the
 * reference's scalar form.  On `stream` (a cudaStream_t, NULL = default stream).  Replaces the CPU rerank of
 * vm-ranker. */
phx_status phx_dpp_rescore_device(int32_t device, const phx_dpp_config* cfg, const phx_dpp_inputs* in, int32_t* out_index,
                                  double* out_score, int32_t* out_count, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PHOENIX_B200_H_ */
