// C ABI of the Phoenix B200 engine (include/phoenix_b200.h): owns weights, the unified embedding
// table and work space, and sequences the kernels of one ranking forward / user-tower pass on one
// stream.  Mirrors the model runner's gather -> forward -> reply sequence
// (phoenix/xrex/inference/model_runner.py:4141-4222) and the model's forward
// (phoenix/xrex/models/recsys_model.py:6082-6224 -> 4734-4883, transformer.py:461-618).
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <vector>

#include "comm.cuh"
#include "common.cuh"

namespace phx {

static std::mutex g_err_mu;
static std::string g_err = "";
void set_global_error(const std::string& msg) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  g_err = msg;
}

static std::atomic<long long> g_dispatch[DK_COUNT];
void dispatch_note(int kind) {
  if (kind >= 0 && kind < DK_COUNT) g_dispatch[kind].fetch_add(1, std::memory_order_relaxed);
}

static inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN
  uint32_t r = ((u >> 16) & 1u) + 0x7FFFu;
  return (uint16_t)((u + r) >> 16);
}
static inline float bf16_bits_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

struct Layer {
  float* pre_attn_norm = nullptr;
  float* pre_ffn_norm = nullptr;
  float* post_attn_norm = nullptr;
  float* post_ffn_norm = nullptr;
  float* q_norm = nullptr;
  float* k_norm = nullptr;
  bf16* w_qkv_f = nullptr;   // [QW, D] with the pre-attention norm gain folded in
  bf16* w_up_f = nullptr;    // [F, D] with the pre-FFN norm gain folded in
  bf16* w_qkv_t = nullptr;   // [QW, D]
  bf16* w_out_t = nullptr;   // [D, HD]
  bf16* w_up_t = nullptr;    // [F, D]
  bf16* w_down_t = nullptr;  // [D, F]
  GemmPlan p_qkv, p_out, p_up, p_down;
  GemmPlan p_qkv_f, p_up_f;  // fused-norm variants: A = residual stream, folded weights
};

}  // namespace phx

using namespace phx;

struct phx_engine {
  struct PackState {
    int *hist_off = nullptr, *cand_off = nullptr, *pos_rows = nullptr, *out_index = nullptr;   // device, owned
    const int *hist_off_view = nullptr, *cand_off_view = nullptr;   // offsets living in a staging block instead
    long long M = 0, Mh = 0;      // packed rows in all, history rows
    int planned_batch = -1;       // batch size pos_rows / out_index were last planned for (full plan)
    bool ragged = false;
  };
  phx_model_config cfg;
  int device = 0;
  int num_sms = 148;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::string err;
  bool use_simt_gemm = false;

  // dimensions
  int D, S, C, T, Hq, Hkv, dh, F, QW, HD, V, NC;
  long long table_rows = 0;        // rows of the whole unified table
  int table_world = 1, table_rank = 0;
  long long shard_rows = 0;        // rows per shard (== table_rows when not sharded)
  const bf16* shard_ptr[PHX_MAX_SHARDS] = {nullptr};   // this device's view of every shard
  void* ipc_opened[PHX_MAX_SHARDS] = {nullptr};
  long long max_tokens = 0;
  // candidate-only tail layers (ranking forward): token rows in split layout, the last n_tail layers update the
  // candidate block only
  bool split = false;
  int n_tail = 0;
  // packed rows (cfg.pack_ragged): every forward addresses its token rows through a PackMap; `full` covers all slots
  // of every request (device-pointer entry points, batches that are not front-filled), `ragged` the counts the
  // host-buffer call found in its batch
  bool pack = false;
  PackState pack_full, pack_ragged;
  PackState pack_device;            // plan handed over by phx_rank_forward_packed_device (offsets in the caller's memory)
  PackState* pack_next = nullptr;   // set by the host-buffer call for the forward it is about to enqueue
  PackState* cur_pack = nullptr;    // the forward being enqueued
  std::vector<int> pack_host;       // host copy of the offsets of the ragged plan
  // projected tokens (cfg.token_project): gathered rows side by side, two projection GEMMs, then scaling
  bool project = false;
  int Kh = 0, Kc = 0;                              // (2H + 2) * D and 2H * D
  bf16 *proj_hist_t = nullptr, *proj_cand_t = nullptr;   // [D, Kh], [D, Kc]
  bf16 *cat_hist = nullptr, *cat_cand = nullptr, *tok_proj = nullptr;   // [max_batch*S, Kh], [max_batch*C, Kc], [max_tokens, D]
  GemmPlan p_proj_hist, p_proj_cand;
  // batch-prep buffers beyond posts and authors (cfg.user_prefix, cand_surface, num_hist_continuous): S counts the
  // user-prefix token, Sh is the number of history slots of the input arrays
  int P = 0, Sh = 0;
  bool prep_extras = false;                        // any of the three: only phx_rank_forward_prep* serves the engine
  int Ku = 0;                                      // user.num_hashes * D
  bf16 *proj_user_t = nullptr, *cat_user = nullptr;   // [D, Ku], [max_batch, Ku]
  GemmPlan p_proj_user;
  bf16* cont_w1[PHX_MAX_HIST_CONT] = {nullptr, nullptr, nullptr, nullptr};
  bf16* cont_w2[PHX_MAX_HIST_CONT] = {nullptr, nullptr, nullptr, nullptr};
  // full-precision path (cfg.compute_fp32): fp32 activations, plain row order
  bool fp32 = false;
  float *x32 = nullptr, *h32 = nullptr, *qkv32 = nullptr, *attn32 = nullptr, *ffn32 = nullptr, *tmp32 = nullptr, *hist32 = nullptr;

  // parameters
  bf16* table = nullptr;
  bf16* action_table = nullptr;
  bf16* surface_table = nullptr;
  float* final_norm = nullptr;
  bf16* unembed_t = nullptr;  // [V+NC, D]
  std::vector<Layer> layers;
  std::map<std::string, bool> loaded;
  float *cos_tab = nullptr, *sin_tab = nullptr;
  phx_blend_spec blend;
  bool has_blend = false;

  // work space
  bf16 *x = nullptr, *hbuf = nullptr, *qkv = nullptr, *attn = nullptr, *ffn = nullptr, *tmp = nullptr, *tokens = nullptr;
  int* seg = nullptr;
  float* rowss_a = nullptr;  // [tokens, D/64] sum-of-squares partials of the rows entering the attention block
  float* rowss_f = nullptr;  // ... entering the FFN block
  bool fused_norm = false;   // RMSNorm folded into the GEMMs (no primer norm, no qk-norm-before-fusion issue, tcgen05 path)
  bool folded_dirty = true;
  int* hashes = nullptr;
  int* err_flag = nullptr;
  // staging for the host-buffer entry point
  void* in_stage_dev = nullptr;
  void* in_stage_host = nullptr;
  size_t in_stage_bytes = 0;
  float* lp_dev = nullptr; float* cont_dev = nullptr; double* score_dev = nullptr;
  float* lp_host = nullptr; float* cont_host = nullptr; double* score_host = nullptr;

  // token prefetch (phx_rank_prefetch_device): tokens of the next batch are built on a side stream into the
  // alternate residual buffer while the current forward runs
  cudaStream_t side_stream = nullptr;
  cudaEvent_t ev_prefetch = nullptr;
  cudaEvent_t ev_chunk[4] = {nullptr, nullptr, nullptr, nullptr};   // result chunks of the host-buffer call
  // two-deep pipeline of host-buffer requests (phx_rank_submit / phx_rank_collect): per slot its own staging blocks
  // and events; the copies run on their own stream so that they overlap the forward of the other slot
  struct StageSlot {
    void* in_dev = nullptr; void* in_host = nullptr;
    float* lp_dev = nullptr; float* cont_dev = nullptr; double* score_dev = nullptr;
    float* lp_host = nullptr; float* cont_host = nullptr; double* score_host = nullptr;
    cudaEvent_t in_ready = nullptr, fwd_done = nullptr, out_done = nullptr;
    cudaEvent_t chunk[4] = {nullptr, nullptr, nullptr, nullptr};
    bool busy = false;
    int batch = 0;
    PackState pack;                 // packed rows of the request in this slot (offset arrays inside the slot's block)
    std::vector<int> pack_host;
  };
  StageSlot slots[2];
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t ev_done[2] = {nullptr, nullptr};   // ends of the last two forwards; done_idx = the most recent
  int done_idx = 0;
  bf16* x_alt = nullptr; int* seg_alt = nullptr; float* rowss_a_alt = nullptr;
  bool prefetch_valid = false;
  phx_rank_batch prefetch_key;

  // CUDA graph of the forward: a call that repeats the previous call's batch size and buffers is captured once and
  // replayed afterwards (the forward is ~42 launches; at small batches their launch gaps are most of its time)
  bool graphs_enabled = true;
  cudaGraphExec_t graph_exec = nullptr;
  bool graph_key_valid = false;
  phx_rank_batch graph_key_b;
  phx_rank_out graph_key_o;
  int graph_launches = 0;
  unsigned long long* gemm_counters = nullptr;   // PHX_GEMM_COUNTERS: [role][total, operand wait, accumulator wait]
  int last_batch = 0;
  int last_launches = 0;
  bool debug_taps = false;
  bool sync_debug = false;

  // optional per-kernel-class timing (phx_profile_enable): events around every launch
  bool profile = false;
  std::vector<std::pair<int, std::pair<cudaEvent_t, cudaEvent_t>>> prof_events;  // (class, (start, stop))
  size_t prof_used = 0;
  cudaEvent_t marks[8] = {};
};

namespace {
enum KernelClass { KC_TOKENS = 0, KC_NORM = 1, KC_GEMM = 2, KC_ROPE = 3, KC_ATTN = 4, KC_HEADS = 5, KC_COUNT = 6 };
struct ProfScope {
  phx_engine* e; cudaEvent_t stop = nullptr;
  ProfScope(phx_engine* e_, int cls) : e(e_), cls_(cls) {
    if (!e->profile) return;
    if (e->prof_used == e->prof_events.size()) {
      cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
      e->prof_events.push_back({cls, {a, b}});
    }
    auto& pe = e->prof_events[e->prof_used++];
    pe.first = cls;   // low byte: kernel class; next byte: optional sub-class
    cudaEventRecord(pe.second.first, e->stream);
    stop = pe.second.second;
  }
  ~ProfScope() {
    if (stop) cudaEventRecord(stop, e->stream);
    if (e->sync_debug) {   // PHX_SYNC_DEBUG=1: find the launch an asynchronous error belongs to
      cudaError_t ce = cudaStreamSynchronize(e->stream);
      if (ce != cudaSuccess)
        fprintf(stderr, "[phx sync-debug] launch #%d (kernel class %d): %s\n", e->last_launches, cls_ & 0xff, cudaGetErrorString(ce));
    }
  }
  int cls_ = -1;
};
}  // namespace

namespace {

template <typename Tp>
phx_status dev_alloc(phx_engine* e, Tp** p, size_t count) {
  PHX_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(Tp)), e->err);
  return PHX_OK;
}

HashFamilyDev to_dev(const phx_hash_family& f, int offset) {
  HashFamilyDev d;
  for (int i = 0; i < PHX_MAX_HASHES; ++i) { d.scales[i] = f.scales[i]; d.biases[i] = f.biases[i]; }
  d.modulus = f.modulus;
  d.buckets_m1 = f.table_size - 1;
  d.magic_mod = f.modulus > 0 ? 0xFFFFFFFFFFFFFFFFull / (unsigned long long)f.modulus : 0;
  d.magic_bkt = d.buckets_m1 > 0 ? 0xFFFFFFFFFFFFFFFFull / (unsigned long long)d.buckets_m1 : 0;
  d.offset = offset;
  d.num_hashes = f.num_hashes;
  return d;
}

PackMap pack_map(const phx_engine::PackState* ps) {
  PackMap m;
  if (ps) {
    m.hist_off = ps->hist_off_view ? ps->hist_off_view : ps->hist_off;
    m.cand_off = ps->cand_off_view ? ps->cand_off_view : ps->cand_off;
    m.cand_base = ps->Mh;
  }
  return m;
}

TableView table_view(const phx_engine* e) {
  TableView v;
  for (int i = 0; i < PHX_MAX_SHARDS; ++i) v.base[i] = e->shard_ptr[i];
  v.total_rows = e->table_rows;
  v.rows_per_shard = (unsigned int)e->shard_rows;
  v.world = e->table_world;
  return v;
}
bool shards_complete(phx_engine* e) {
  for (int i = 0; i < e->table_world; ++i)
    if (!e->shard_ptr[i]) { e->err = "table shard " + std::to_string(i) + " is not attached (phx_table_attach_peer)"; return false; }
  return true;
}

// region offsets of the unified table: phoenix/xrex/models/recsys_embedding.py:234-248
void region_offsets(const phx_model_config& c, long long* user, long long* item, long long* author, long long* ip,
                    long long* total) {
  *user = 1 + 64;
  *item = *user + c.user.table_size;
  *author = *item + c.item.table_size;
  *ip = *author + c.author.table_size;
  *total = *ip + c.ip.table_size;
}

phx_status check_cfg(const phx_model_config& c, std::string& err) {
  auto bad = [&](const char* m) { err = std::string("config: ") + m; return PHX_E_ARG; };
  if (c.emb_size <= 0 || c.emb_size % 64 != 0) return bad("emb_size must be a positive multiple of 64");
  if (c.key_size != 32 && c.key_size != 64 && c.key_size != 128) return bad("key_size must be 32, 64 or 128");
  if (c.num_q_heads <= 0 || c.num_kv_heads <= 0 || c.num_q_heads % c.num_kv_heads != 0) return bad("head counts");
  if (c.ffn_size <= 0 || c.ffn_size % 64 != 0) return bad("ffn_size must be a positive multiple of 64");
  if (c.num_layers <= 0 || c.history_len <= 0 || c.num_candidates < 0 || c.max_batch <= 0) return bad("sizes");
  if (c.num_actions < 0 || c.num_continuous < 0 || c.num_actions + c.num_continuous > 32) return bad("at most 32 heads");
  if (c.num_candidates > 0 && c.num_actions + c.num_continuous == 0) return bad("ranking engine needs heads");
  const phx_hash_family* fams[4] = {&c.user, &c.item, &c.author, &c.ip};
  for (auto f : fams) {
    if (f->num_hashes < 0 || f->num_hashes > PHX_MAX_HASHES) return bad("num_hashes out of range");
    if (f->table_size < 0 || (f->num_hashes > 0 && (f->table_size < 2 || f->modulus <= 0))) return bad("hash family");
  }
  if (c.item.num_hashes <= 0 || c.item.num_hashes != c.author.num_hashes) return bad("item/author hash counts must match");
  if (c.cap_method < 0 || c.cap_method > 2) return bad("cap_method");
  if (c.table_world < 0 || c.table_world > PHX_MAX_SHARDS || (c.table_world > 1 && (c.table_rank < 0 || c.table_rank >= c.table_world)))
    return bad("table_world / table_rank");
  if (c.compute_fp32 != 0 && c.compute_fp32 != 1) return bad("compute_fp32 must be 0 or 1");
  if (c.token_project != 0 && c.token_project != 1) return bad("token_project must be 0 or 1");
  if (c.token_project && c.compute_fp32) return bad("projected tokens are not available on the full-precision path");
  if (c.pack_ragged != 0 && c.pack_ragged != 1) return bad("pack_ragged must be 0 or 1");
  if (c.action_multi_hot != 0 && c.action_multi_hot != 1) return bad("action_multi_hot must be 0 or 1");
  if (c.action_multi_hot && (c.num_action_types < 1 || c.num_action_types > 32 || c.emb_size % c.num_action_types != 0 ||
                             (c.emb_size / c.num_action_types) % 8 != 0))
    return bad("action sets need 1..32 action types and emb_size / num_action_types a multiple of 8");
  if (c.pack_ragged && c.compute_fp32) return bad("packed rows are not available on the full-precision path");
  if (c.num_candidate_only_layers < 0 || c.num_candidate_only_layers > c.num_layers) return bad("num_candidate_only_layers");
  if ((c.user_prefix != 0 && c.user_prefix != 1) || (c.cand_surface != 0 && c.cand_surface != 1)) return bad("user_prefix / cand_surface must be 0 or 1");
  if (c.user_prefix && (c.num_candidates <= 0 || c.user.num_hashes <= 0 || c.user.num_hashes + c.ip.num_hashes > 2 * PHX_MAX_HASHES))
    return bad("user_prefix needs a ranking engine and 1..PHX_MAX_HASHES user hashes");
  if (c.cand_surface && c.num_candidates <= 0) return bad("cand_surface needs candidates");
  if (c.num_hist_continuous < 0 || c.num_hist_continuous > PHX_MAX_HIST_CONT) return bad("num_hist_continuous out of range");
  if (c.num_hist_continuous > 0 && c.hist_cont_hidden != 32 && c.hist_cont_hidden != 64) return bad("hist_cont_hidden must be 32 or 64");
  for (int i = 0; i < c.num_hist_continuous; ++i)
    if (c.hist_cont_index[i] < 0 || c.hist_cont_index[i] >= PHX_PREP_CONTINUOUS || !(c.hist_cont_norm_scale[i] > 0.f))
      return bad("hist_cont_index / hist_cont_norm_scale");
  if ((c.user_prefix || c.cand_surface || c.num_hist_continuous > 0) && (c.pack_ragged || c.table_world > 1))
    return bad("user_prefix / cand_surface / continuous history actions are not available with packed rows or a sharded table");
  return PHX_OK;
}

phx_status upload_f32(phx_engine* e, float** dst, const float* host, size_t n, bool round_bf16) {
  std::vector<float> tmp(host, host + n);
  if (round_bf16) for (auto& v : tmp) v = bf16_bits_to_f32(f32_to_bf16_bits(v));
  if (!*dst) { phx_status s = dev_alloc(e, dst, n); if (s) return s; }
  PHX_CUDA_TRY(cudaMemcpy(*dst, tmp.data(), n * sizeof(float), cudaMemcpyHostToDevice), e->err);
  return PHX_OK;
}
// host [rows, cols] f32 (in, out) -> device bf16; transposed to [cols, rows] when `transpose`
phx_status upload_bf16(phx_engine* e, bf16** dst, const float* host, int64_t rows, int64_t cols, bool transpose) {
  std::vector<uint16_t> tmp((size_t)rows * cols);
  if (transpose) {
    for (int64_t r = 0; r < rows; ++r)
      for (int64_t c = 0; c < cols; ++c) tmp[(size_t)c * rows + r] = f32_to_bf16_bits(host[(size_t)r * cols + c]);
  } else {
    for (size_t i = 0; i < tmp.size(); ++i) tmp[i] = f32_to_bf16_bits(host[i]);
  }
  if (!*dst) { phx_status s = dev_alloc(e, dst, tmp.size()); if (s) return s; }
  PHX_CUDA_TRY(cudaMemcpy(*dst, tmp.data(), tmp.size() * 2, cudaMemcpyHostToDevice), e->err);
  return PHX_OK;
}

phx_status do_gemm(phx_engine* e, GemmPlan& p, const bf16* A, bf16* Cc, const bf16* R, int64_t M, int epi,
                   const GemmRope* rope = nullptr, const GemmNorm* norm = nullptr) {
  ProfScope ps(e, KC_GEMM | ((epi + 1) << 8));   // sub-class = epilogue, for the optional per-GEMM breakdown
  e->last_launches++;
  if (e->use_simt_gemm) return gemm_simt_launch(A, p.Wt, Cc, R, M, p.N, p.K, epi, e->stream, e->err);
  return gemm_launch(p, A, Cc, R, M, epi, rope, norm, e->err_flag, e->num_sms, e->stream, e->err);
}

// fold the norm gains into the weights of the GEMMs that consume the normed rows (after any parameter reload)
phx_status refresh_folded(phx_engine* e) {
  if (!e->fused_norm || !e->folded_dirty) return PHX_OK;
  for (auto& L : e->layers) {
    phx_status s;
    if ((s = fold_gain_launch(L.w_qkv_t, L.pre_attn_norm, L.w_qkv_f, e->QW, e->D, e->stream, e->err))) return s;
    if ((s = fold_gain_launch(L.w_up_t, L.pre_ffn_norm, L.w_up_f, e->F, e->D, e->stream, e->err))) return s;
  }
  e->folded_dirty = false;
  return PHX_OK;
}

bool params_complete(phx_engine* e, bool need_heads) {
  std::vector<std::string> need = {"action_table", "surface_table", "final_norm"};
  if (e->project) { need.push_back("proj_hist"); if (need_heads) need.push_back("proj_cand"); if (e->P) need.push_back("proj_user"); }
  for (int i = 0; i < e->cfg.num_hist_continuous; ++i) {
    need.push_back("hist_cont" + std::to_string(i) + ".proj1"); need.push_back("hist_cont" + std::to_string(i) + ".proj2");
  }
  if (need_heads) {
    if (e->V > 0) need.push_back("unembed");
    if (e->NC > 0) need.push_back("cont_unembed");
  }
  for (int l = 0; l < e->cfg.num_layers; ++l) {
    std::string p = "layer" + std::to_string(l) + ".";
    for (const char* n : {"pre_attn_norm", "w_qkv", "w_out", "pre_ffn_norm", "w_up", "w_down"}) need.push_back(p + n);
    if (e->cfg.qk_norm) { need.push_back(p + "q_norm"); need.push_back(p + "k_norm"); }
    if (e->cfg.primer_norm) { need.push_back(p + "post_attn_norm"); need.push_back(p + "post_ffn_norm"); }
  }
  for (auto& n : need)
    if (!e->loaded.count(n)) { e->err = "parameter not loaded: " + n; return false; }
  return true;
}

// The same layers in fp32 (fp32_path.cu), rows in plain [B, Tt] order.  A candidate-only tail is done the way the
// reference's non-kernel path does it (transformer.py:848-858): the layer runs over every row, then the history rows
// are put back to their values at the tail's entrance.
phx_status run_trunk_f32(phx_engine* e, int B, int Tt, int pos_cap, int hist_len, int n_tail) {
  const long long M = (long long)B * Tt;
  const phx_model_config& c = e->cfg;
  const float sm_scale = sqrtf(128.0f) / (float)c.key_size;
  const size_t hist_bytes = (size_t)hist_len * e->D * sizeof(float), row_bytes = (size_t)Tt * e->D * sizeof(float);
  phx_status s;
  auto gemm = [&](const float* A, const bf16* Wt, float* Cc, const float* R, int N, int K, int epi) {
    ProfScope ps(e, KC_GEMM | ((epi + 1) << 8));
    e->last_launches++;
    return f32_gemm_launch(A, Wt, Cc, R, M, N, K, epi, e->stream, e->err);
  };
  auto norm = [&](const float* x, const float* gain, float* y, const float* res) {
    ProfScope ps(e, KC_NORM);
    e->last_launches++;
    return f32_rmsnorm_launch(x, gain, y, res, M, e->D, c.rms_eps, e->stream, e->err);
  };
  for (int l = 0; l < c.num_layers; ++l) {
    Layer& L = e->layers[l];
    const bool tail = n_tail > 0 && l >= c.num_layers - n_tail;
    if (tail && l == c.num_layers - n_tail)
      PHX_CUDA_TRY(cudaMemcpy2DAsync(e->hist32, hist_bytes, e->x32, row_bytes, hist_bytes, B, cudaMemcpyDeviceToDevice, e->stream), e->err);
    if ((s = norm(e->x32, L.pre_attn_norm, e->h32, nullptr))) return s;
    if ((s = gemm(e->h32, L.w_qkv_t, e->qkv32, nullptr, e->QW, e->D, EPI_STORE))) return s;
    if (c.rotary || c.qk_norm) {
      ProfScope ps(e, KC_ROPE);
      e->last_launches++;
      if ((s = f32_qknorm_rope_launch(e->qkv32, M, Tt, e->Hq, e->Hkv, e->dh, pos_cap, c.rotary, c.qk_norm, L.q_norm, L.k_norm,
                                      e->cos_tab, e->sin_tab, e->stream, e->err))) return s;
    }
    { ProfScope ps(e, KC_ATTN);
      e->last_launches++;
      if ((s = f32_attention_launch(e->qkv32, e->seg, e->attn32, B, Tt, e->Hq, e->Hkv, e->dh, hist_len, sm_scale, c.attn_logit_cap,
                                    (c.attn_logit_cap > 0.f) ? c.cap_method : 0, e->stream, e->err))) return s; }
    if (c.primer_norm) {
      if ((s = gemm(e->attn32, L.w_out_t, e->tmp32, nullptr, e->D, e->HD, EPI_STORE))) return s;
      if ((s = norm(e->tmp32, L.post_attn_norm, e->x32, e->x32))) return s;
    } else {
      if ((s = gemm(e->attn32, L.w_out_t, e->x32, e->x32, e->D, e->HD, EPI_RESIDUAL))) return s;
    }
    if ((s = norm(e->x32, L.pre_ffn_norm, e->h32, nullptr))) return s;
    if ((s = gemm(e->h32, L.w_up_t, e->ffn32, nullptr, e->F, e->D, EPI_GELU))) return s;
    if (c.primer_norm) {
      if ((s = gemm(e->ffn32, L.w_down_t, e->tmp32, nullptr, e->D, e->F, EPI_STORE))) return s;
      if ((s = norm(e->tmp32, L.post_ffn_norm, e->x32, e->x32))) return s;
    } else {
      if ((s = gemm(e->ffn32, L.w_down_t, e->x32, e->x32, e->D, e->F, EPI_RESIDUAL))) return s;
    }
    if (tail)
      PHX_CUDA_TRY(cudaMemcpy2DAsync(e->x32, row_bytes, e->hist32, hist_bytes, hist_bytes, B, cudaMemcpyDeviceToDevice, e->stream), e->err);
  }
  return PHX_OK;
}

// trunk over `Tt` tokens per request (history + candidates, or history only for the tower).
// split: the rows are in split layout (token_row); the last `n_tail` layers then update the candidate rows only
// (transformer.py:789-871): their QKV projection still covers every row - the history keys / values of a tail layer
// come from the frozen history rows through that layer's own norm and weights (layers.py:608-619) - while attention
// (queries), out-projection and FFN run over the contiguous candidate block.
phx_status run_trunk(phx_engine* e, int B, int Tt, int pos_cap, int hist_len, bool split = false, int n_tail = 0) {
  if (e->fp32) return run_trunk_f32(e, B, Tt, pos_cap, hist_len, n_tail);
  const phx_engine::PackState* pk = split ? nullptr : e->cur_pack;   // packed rows (ranking forward of a packing engine)
  const long long M = pk ? pk->M : (long long)B * Tt;
  const phx_model_config& c = e->cfg;
  const float sm_scale = sqrtf(128.0f) / (float)c.key_size;  // phoenix/xrex/models/scaling.py:46-47
  phx_status s;
  for (int l = 0; l < c.num_layers; ++l) {
    Layer& L = e->layers[l];
    const bool fused = e->fused_norm;
    const int slots = e->D / 64;
    const bool tail = (split || pk) && l >= c.num_layers - n_tail;
    const long long off = tail ? (pk ? pk->Mh : (long long)B * hist_len) : 0;   // first row the out-projection and FFN update
    const long long Mu = M - off;                                // rows they update
    GemmNorm n_attn_in = {e->rowss_a, nullptr, slots, 1.0f / (float)e->D, c.rms_eps};   // consume stats of x -> QKV
    GemmNorm n_attn_out = {nullptr, e->rowss_f ? e->rowss_f + off * slots : nullptr, 0, 0.f, 0.f};   // out-proj leaves stats for the FFN
    GemmNorm n_ffn_in = {e->rowss_f ? e->rowss_f + off * slots : nullptr, nullptr, slots, 1.0f / (float)e->D, c.rms_eps};
    GemmNorm n_ffn_out = {nullptr, e->rowss_a ? e->rowss_a + off * slots : nullptr, 0, 0.f, 0.f};    // down-proj leaves stats for the next layer
    if (!fused) {
      { ProfScope ps(e, KC_NORM);
      if ((s = rmsnorm_launch(e->x, L.pre_attn_norm, e->hbuf, nullptr, M, e->D, c.rms_eps, e->stream, e->err))) return s; }
      e->last_launches++;
    }
    GemmPlan& pq = fused ? L.p_qkv_f : L.p_qkv;
    GemmPlan& pu = fused ? L.p_up_f : L.p_up;
    const bf16* a_in = fused ? e->x : e->hbuf;
    // RoPE rides in the QKV epilogue unless qk-norm has to run first or the head dim is 128
    const bool fuse_rope = c.rotary && !c.qk_norm && !e->use_simt_gemm && (e->dh == 32 || e->dh == 64);
    if (fuse_rope) {
      GemmRope gr;
      gr.cos_tab = e->cos_tab; gr.sin_tab = e->sin_tab; gr.T = Tt; gr.pos_cap = pos_cap; gr.dh = e->dh;
      gr.g = e->Hq / e->Hkv; gr.group = gr.g + 2;
      if (split) { gr.T = hist_len; gr.split_rows = (long long)B * hist_len; }
      if (pk) gr.pos_rows = pk->pos_rows;
      if ((s = do_gemm(e, pq, a_in, e->qkv, nullptr, M, EPI_ROPE, &gr, fused ? &n_attn_in : nullptr))) return s;
    } else {
      if ((s = do_gemm(e, pq, a_in, e->qkv, nullptr, M, EPI_STORE, nullptr, fused ? &n_attn_in : nullptr))) return s;
    }
    if (!fuse_rope && (c.rotary || c.qk_norm)) {
      QkNormRopeArgs qa;
      qa.qkv = e->qkv; qa.M = M; qa.T = Tt; qa.Hq = e->Hq; qa.Hkv = e->Hkv; qa.dh = e->dh; qa.pos_cap = pos_cap;
      qa.rotary = c.rotary; qa.qk_norm = c.qk_norm; qa.q_gain = L.q_norm; qa.k_gain = L.k_norm;
      qa.cos_tab = e->cos_tab; qa.sin_tab = e->sin_tab;
      if (split) { qa.T = hist_len; qa.split_rows = (long long)B * hist_len; }
      if (pk) qa.pos_rows = pk->pos_rows;
      { ProfScope ps(e, KC_ROPE); if ((s = qknorm_rope_launch(qa, e->stream, e->err))) return s; }
      e->last_launches++;
    }
    AttnArgs aa;
    const int g = e->Hq / e->Hkv;
    aa.q = e->qkv; aa.k = e->qkv + (long long)g * e->dh; aa.v = e->qkv + (long long)(g + 1) * e->dh;
    aa.q_tok_stride = aa.k_tok_stride = aa.v_tok_stride = e->QW;
    // merged QKV row: per kv head [q_0..q_{g-1}, k, v] (layers.py:728-736): q head h sits at column
    // ((h / g) * (g + 2) + h % g) * dh, kv head j's k at (j * (g + 2) + g) * dh
    aa.q_head_stride = (g == 1) ? (g + 2) * e->dh : e->dh;
    aa.q_group = g; aa.q_group_stride = (g + 2) * e->dh;
    aa.k_head_stride = (g + 2) * e->dh; aa.v_head_stride = (g + 2) * e->dh;
    aa.out = e->attn; aa.seg = e->seg; aa.B = B; aa.T = Tt; aa.Hq = e->Hq; aa.Hkv = e->Hkv; aa.dh = e->dh;
    aa.hist_len = hist_len; aa.sm_scale = sm_scale; aa.cap = c.attn_logit_cap;
    aa.cap_method = (c.attn_logit_cap > 0.f) ? c.cap_method : 0;
    aa.err_flag = e->err_flag;
    aa.split = split ? 1 : 0; aa.q_start = tail ? hist_len : 0;
    aa.pack = pack_map(pk);
    { ProfScope ps(e, KC_ATTN); if ((s = ranker_attention_launch(aa, e->stream, e->err))) return s; }
    e->last_launches++;
    if (Mu == 0) continue;                              // a candidate-only layer of a batch without candidates
    bf16* xu = e->x + off * e->D;                       // the rows this layer updates
    const bf16* attn_u = e->attn + off * e->HD;
    bf16* ffn_u = e->ffn + off * e->F;
    if (c.primer_norm) {
      // x = x + post_attn_norm(out(attn)) (transformer.py:531-541)
      if ((s = do_gemm(e, L.p_out, attn_u, e->tmp, nullptr, Mu, EPI_STORE))) return s;
      { ProfScope ps(e, KC_NORM); if ((s = rmsnorm_launch(e->tmp, L.post_attn_norm, xu, xu, Mu, e->D, c.rms_eps, e->stream, e->err))) return s; }
      e->last_launches++;
    } else {
      if ((s = do_gemm(e, L.p_out, attn_u, xu, xu, Mu, EPI_RESIDUAL, nullptr, fused ? &n_attn_out : nullptr))) return s;
    }
    if (!fused) {
      { ProfScope ps(e, KC_NORM); if ((s = rmsnorm_launch(xu, L.pre_ffn_norm, e->hbuf, nullptr, Mu, e->D, c.rms_eps, e->stream, e->err))) return s; }
      e->last_launches++;
    }
    if ((s = do_gemm(e, pu, fused ? xu : e->hbuf, ffn_u, nullptr, Mu, EPI_GELU, nullptr, fused ? &n_ffn_in : nullptr))) return s;
    if (c.primer_norm) {
      if ((s = do_gemm(e, L.p_down, ffn_u, e->tmp, nullptr, Mu, EPI_STORE))) return s;
      { ProfScope ps(e, KC_NORM); if ((s = rmsnorm_launch(e->tmp, L.post_ffn_norm, xu, xu, Mu, e->D, c.rms_eps, e->stream, e->err))) return s; }
      e->last_launches++;
    } else {
      if ((s = do_gemm(e, L.p_down, ffn_u, xu, xu, Mu, EPI_RESIDUAL, nullptr, fused ? &n_ffn_out : nullptr))) return s;
    }
  }
  return PHX_OK;
}

// Pre-hashed input of one forward, device pointers: phx_rank_batch_hashed or phx_rank_batch_prep brought to one form.
struct HashedIn {
  const int *hist_post = nullptr, *hist_author = nullptr, *cand_post = nullptr, *cand_author = nullptr;
  const int *hist_actions = nullptr, *hist_surfaces = nullptr, *cand_surfaces = nullptr;
  const unsigned char* hist_actions_bool = nullptr;
  const int *user_hashes = nullptr, *user_ip_hashes = nullptr;
  const float* hist_cont = nullptr;
};

phx_status build_tokens(phx_engine* e, const phx_rank_batch* bd, int B, int Cc, bf16* x_dst = nullptr, int* seg_dst = nullptr,
                        cudaStream_t stream = nullptr, float* ss_dst = nullptr, int* rows_out = nullptr,
                        const bf16* landing = nullptr, const int* pos = nullptr, const HashedIn* hb = nullptr) {
  long long ou, oi, oa, oip, tot;
  region_offsets(e->cfg, &ou, &oi, &oa, &oip, &tot);
  TokenBuildArgs ta;
  if (hb) {   // rows already hashed by the host's batch-prep (bd is not read)
    ta.hist_post = ta.hist_author = ta.cand_post = ta.cand_author = nullptr;
    ta.pre_hist_post = hb->hist_post; ta.pre_hist_author = hb->hist_author;
    ta.pre_cand_post = hb->cand_post; ta.pre_cand_author = hb->cand_author;
    ta.hist_actions = hb->hist_actions; ta.hist_surfaces = hb->hist_surfaces;
    ta.hist_actions_bool = hb->hist_actions_bool;
    if (e->cfg.cand_surface) ta.cand_surfaces = hb->cand_surfaces;
    if (e->P) {
      ta.P = e->P; ta.Hu = e->cfg.user.num_hashes; ta.Hip = e->cfg.ip.num_hashes;
      ta.user_hashes = hb->user_hashes; ta.user_ip_hashes = ta.Hip > 0 ? hb->user_ip_hashes : nullptr;
    }
    if (e->cfg.num_hist_continuous > 0) {
      ta.hist_cont = hb->hist_cont; ta.n_cont = e->cfg.num_hist_continuous; ta.cont_hidden = e->cfg.hist_cont_hidden;
      for (int i = 0; i < ta.n_cont; ++i) {
        ta.cont_index[i] = e->cfg.hist_cont_index[i]; ta.cont_log[i] = e->cfg.hist_cont_use_log[i];
        ta.cont_scale[i] = e->cfg.hist_cont_norm_scale[i]; ta.cont_w1[i] = e->cont_w1[i]; ta.cont_w2[i] = e->cont_w2[i];
      }
    }
  } else {
    ta.hist_post = (const long long*)bd->hist_post_ids; ta.hist_author = (const long long*)bd->hist_author_ids;
    ta.hist_actions = bd->hist_actions; ta.hist_surfaces = bd->hist_surfaces;
    ta.cand_post = (const long long*)bd->cand_post_ids; ta.cand_author = (const long long*)bd->cand_author_ids;
  }
  ta.table = table_view(e);
  ta.action_table = e->action_table; ta.surface_table = e->surface_table;
  ta.num_action_types = e->cfg.num_action_types; ta.num_surfaces = e->cfg.num_surfaces;
  ta.action_multi_hot = e->cfg.action_multi_hot;
  ta.item = to_dev(e->cfg.item, (int)oi); ta.author = to_dev(e->cfg.author, (int)oa);
  ta.B = B; ta.S = e->S; ta.C = Cc; ta.D = e->D;
  ta.input_scale = sqrtf((float)e->D);  // scaling.py:40-41
  ta.x = x_dst ? x_dst : e->x; ta.tokens = e->debug_taps ? e->tokens : nullptr; ta.hashes = e->debug_taps ? e->hashes : nullptr;
  ta.seg = seg_dst ? seg_dst : e->seg;
  ta.row_ss = e->fused_norm ? (ss_dst ? ss_dst : e->rowss_a) : nullptr;
  ta.ss_slots = e->D / 64;
  ta.split = (e->split && Cc > 0) ? 1 : 0;
  if (e->cur_pack && Cc > 0 && !rows_out) ta.pack = pack_map(e->cur_pack);
  if (e->fp32) ta.x32 = e->x32;
  if (rows_out) { ta.rows_only = 1; ta.hashes = rows_out; }
  ta.landing = landing; ta.pos = pos;
  if (e->project && !rows_out) {
    // gathered rows side by side -> two projection GEMMs -> scale, place and take the row statistics
    if (stream) { e->err = "token prefetch is not available with projected tokens"; return PHX_E_ARG; }
    ta.concat_hist = e->cat_hist; ta.concat_cand = e->cat_cand; ta.concat_user = e->cat_user;
    cudaStream_t st = e->stream;
    phx_status s;
    { e->last_launches++; ProfScope ps(e, KC_TOKENS); if ((s = build_tokens_launch(ta, st, e->err))) return s; }
    bf16* tok_u = e->tok_proj; bf16* tok_h = tok_u + (long long)B * e->P * e->D; bf16* tok_c = tok_h + (long long)B * e->Sh * e->D;
    if (e->P && (s = do_gemm(e, e->p_proj_user, e->cat_user, tok_u, nullptr, (long long)B, EPI_STORE))) return s;
    if ((s = do_gemm(e, e->p_proj_hist, e->cat_hist, tok_h, nullptr, (long long)B * e->Sh, EPI_STORE))) return s;
    if (Cc > 0 && (s = do_gemm(e, e->p_proj_cand, e->cat_cand, tok_c, nullptr, (long long)B * Cc, EPI_STORE))) return s;
    e->last_launches++;
    ProfScope ps(e, KC_TOKENS);
    return finish_tokens_launch(tok_u, tok_h, tok_c, ta, st, e->err);
  }
  if (stream) return build_tokens_launch(ta, stream, e->err);   // prefetch on the side stream: not profiled
  e->last_launches++;
  ProfScope ps(e, KC_TOKENS);
  return build_tokens_launch(ta, e->stream, e->err);
}

phx_status check_err_flag(phx_engine* e) {
  int flag = 0;
  PHX_CUDA_TRY(cudaMemcpy(&flag, e->err_flag, sizeof(int), cudaMemcpyDeviceToHost), e->err);
  if (flag != 0) {
    cudaMemset(e->err_flag, 0, sizeof(int));
    e->err = "a bounded device-side wait ran out (GEMM / attention pipeline)";
    return PHX_E_TIMEOUT;
  }
  return PHX_OK;
}

}  // namespace

extern "C" {

const char* phx_global_error(void) { return g_err.c_str(); }
const char* phx_last_error(const phx_engine* e) { return e ? e->err.c_str() : g_err.c_str(); }

phx_status phx_engine_create(const phx_model_config* cfg, int32_t device, phx_engine** out) {
  if (!cfg || !out) { set_global_error("phx_engine_create: null argument"); return PHX_E_ARG; }
  std::string err;
  phx_status s = check_cfg(*cfg, err);
  if (s) { set_global_error(err); return s; }
  phx_engine* e = new phx_engine();
  e->cfg = *cfg; e->device = device;
  auto fail = [&](phx_status st) { set_global_error(e->err); phx_engine_destroy(e); return st; };
  if (cudaSetDevice(device) != cudaSuccess) { e->err = "cudaSetDevice failed"; return fail(PHX_E_CUDA); }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { e->err = "cudaGetDeviceProperties failed"; return fail(PHX_E_CUDA); }
  if (prop.major != 10) { e->err = "this library is built for sm_100a (B200) only"; return fail(PHX_E_ARG); }
  e->num_sms = prop.multiProcessorCount;
  const char* gi = getenv("PHX_GEMM");
  e->use_simt_gemm = gi && strcmp(gi, "simt") == 0;
  const char* dt = getenv("PHX_DEBUG_TAPS");
  e->debug_taps = dt && dt[0] == '1';
#ifdef PHX_DIAGNOSTICS
  { const char* sd = getenv("PHX_SYNC_DEBUG"); e->sync_debug = sd && sd[0] == '1'; }
#endif
  { const char* g = getenv("PHX_GRAPH"); e->graphs_enabled = !(g && g[0] == '0'); }
  e->P = cfg->user_prefix ? 1 : 0; e->Sh = cfg->history_len;
  e->prep_extras = cfg->user_prefix || cfg->cand_surface || cfg->num_hist_continuous > 0;
  e->D = cfg->emb_size; e->S = e->Sh + e->P; e->C = cfg->num_candidates; e->T = e->S + e->C;
  e->Hq = cfg->num_q_heads; e->Hkv = cfg->num_kv_heads; e->dh = cfg->key_size; e->F = cfg->ffn_size;
  e->QW = (e->Hq + 2 * e->Hkv) * e->dh; e->HD = e->Hq * e->dh; e->V = cfg->num_actions; e->NC = cfg->num_continuous;
  long long ou, oi, oa, oip, tot;
  region_offsets(*cfg, &ou, &oi, &oa, &oip, &tot);
  e->table_rows = tot;
  if (tot >= (1ll << 31)) { e->err = "the unified table must have fewer than 2^31 rows"; return fail(PHX_E_ARG); }
  e->table_world = cfg->table_world > 1 ? cfg->table_world : 1;
  e->table_rank = cfg->table_world > 1 ? cfg->table_rank : 0;
  e->shard_rows = (tot + e->table_world - 1) / e->table_world;
  e->max_tokens = (long long)cfg->max_batch * e->T;
  e->n_tail = e->C > 0 ? cfg->num_candidate_only_layers : 0;
  e->fp32 = cfg->compute_fp32 != 0;
  e->pack = cfg->pack_ragged != 0 && e->C > 0;
  // The last layer's history rows are never read again by the ranking forward (the heads take candidate rows, and
  // that layer's history keys / values come from its input), so it can always run as a candidate-only layer with the
  // same candidate outputs bit for bit.  Done wherever the rows can be kept history-first at no cost: packed rows,
  // and the plain engine in the regime its attention runs on the mma.sync kernels anyway (the tcgen05 attention
  // kernel wants [B, T] rows).  PHX_LAST_LAYER=full keeps every row in the last layer.
  {
    const char* ll = getenv("PHX_LAST_LAYER");
    const bool keep_full = ll && strcmp(ll, "full") == 0;
    const bool mma_regime = e->dh != 128 && e->S <= 128;
    if (e->C > 0 && !e->fp32 && !keep_full && e->n_tail == 0 && (e->pack || mma_regime)) e->n_tail = 1;
  }
  e->split = e->n_tail > 0 && !e->fp32 && !e->pack;   // packed rows carry their own history-first order
  const long long M = e->max_tokens;
#define TRY(x) do { phx_status _s = (x); if (_s) return fail(_s); } while (0)
#define CU(x) do { cudaError_t _c = (x); if (_c != cudaSuccess) { e->err = std::string(#x) + ": " + cudaGetErrorString(_c); return fail(PHX_E_CUDA); } } while (0)
  CU(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
  CU(cudaEventCreate(&e->ev0)); CU(cudaEventCreate(&e->ev1));
  TRY(dev_alloc(e, &e->table, (size_t)e->shard_rows * e->D));
  CU(cudaMemset(e->table, 0, (size_t)e->shard_rows * e->D * 2));
  e->shard_ptr[e->table_rank] = e->table;
  TRY(dev_alloc(e, &e->x, (size_t)M * e->D));
  TRY(dev_alloc(e, &e->hbuf, (size_t)M * e->D));
  TRY(dev_alloc(e, &e->qkv, (size_t)M * e->QW));
  TRY(dev_alloc(e, &e->attn, (size_t)M * e->HD));
  TRY(dev_alloc(e, &e->ffn, (size_t)M * e->F));
  TRY(dev_alloc(e, &e->seg, (size_t)M));
  {
    const char* nf = getenv("PHX_NORM");
    e->fused_norm = !cfg->primer_norm && !e->use_simt_gemm && !e->fp32 && !(nf && strcmp(nf, "separate") == 0);
    if (e->fused_norm) {
      TRY(dev_alloc(e, &e->rowss_a, (size_t)M * (e->D / 64)));
      TRY(dev_alloc(e, &e->rowss_f, (size_t)M * (e->D / 64)));
    }
  }
  if (cfg->primer_norm) TRY(dev_alloc(e, &e->tmp, (size_t)M * e->D));
  if (e->pack) {
    const int Bm = cfg->max_batch;
    for (phx_engine::PackState* ps : {&e->pack_full, &e->pack_ragged}) {
      TRY(dev_alloc(e, &ps->hist_off, (size_t)Bm + 1));
      TRY(dev_alloc(e, &ps->cand_off, (size_t)Bm + 1));
      TRY(dev_alloc(e, &ps->pos_rows, (size_t)M));
      TRY(dev_alloc(e, &ps->out_index, (size_t)Bm * e->C));
    }
    std::vector<int> ho(Bm + 1), co(Bm + 1);
    for (int b = 0; b <= Bm; ++b) { ho[b] = b * e->S; co[b] = b * e->C; }
    CU(cudaMemcpy(e->pack_full.hist_off, ho.data(), ho.size() * 4, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(e->pack_full.cand_off, co.data(), co.size() * 4, cudaMemcpyHostToDevice));
    e->pack_ragged.ragged = true;
    e->pack_host.resize(2 * ((size_t)Bm + 1));
  }
  e->project = cfg->token_project != 0;
  if (e->project) {
    const int H2 = 2 * cfg->item.num_hashes;
    e->Kh = (H2 + 2) * e->D; e->Kc = (H2 + (cfg->cand_surface ? 1 : 0)) * e->D;
    const long long mh = (long long)cfg->max_batch * e->Sh, mc = (long long)cfg->max_batch * (e->C > 0 ? e->C : 1);
    if (e->P) {
      e->Ku = cfg->user.num_hashes * e->D;
      TRY(dev_alloc(e, &e->proj_user_t, (size_t)e->D * e->Ku));
      TRY(dev_alloc(e, &e->cat_user, (size_t)cfg->max_batch * e->Ku));
      TRY(gemm_plan_create(&e->p_proj_user, e->cat_user, e->proj_user_t, cfg->max_batch, e->D, e->Ku, false, e->err));
    }
    TRY(dev_alloc(e, &e->proj_hist_t, (size_t)e->D * e->Kh));
    TRY(dev_alloc(e, &e->proj_cand_t, (size_t)e->D * e->Kc));
    TRY(dev_alloc(e, &e->cat_hist, (size_t)mh * e->Kh));
    TRY(dev_alloc(e, &e->cat_cand, (size_t)mc * e->Kc));
    TRY(dev_alloc(e, &e->tok_proj, (size_t)M * e->D));
    TRY(gemm_plan_create(&e->p_proj_hist, e->cat_hist, e->proj_hist_t, mh, e->D, e->Kh, false, e->err));
    TRY(gemm_plan_create(&e->p_proj_cand, e->cat_cand, e->proj_cand_t, mc, e->D, e->Kc, false, e->err));
  }
  if (e->fp32) {
    TRY(dev_alloc(e, &e->x32, (size_t)M * e->D));
    TRY(dev_alloc(e, &e->h32, (size_t)M * e->D));
    TRY(dev_alloc(e, &e->qkv32, (size_t)M * e->QW));
    TRY(dev_alloc(e, &e->attn32, (size_t)M * e->HD));
    TRY(dev_alloc(e, &e->ffn32, (size_t)M * e->F));
    if (cfg->primer_norm) TRY(dev_alloc(e, &e->tmp32, (size_t)M * e->D));
    if (e->n_tail > 0) TRY(dev_alloc(e, &e->hist32, (size_t)cfg->max_batch * e->S * e->D));
  }
  if (e->debug_taps) {
    TRY(dev_alloc(e, &e->tokens, (size_t)M * e->D));
    TRY(dev_alloc(e, &e->hashes, (size_t)M * 2 * cfg->item.num_hashes));
  }
  TRY(dev_alloc(e, &e->err_flag, 2));   // [0] raised by a wait that ran out, [1] the wait limit in microseconds (0 = default)
  CU(cudaMemset(e->err_flag, 0, 2 * sizeof(int)));
  // RoPE tables: angle = pos * base^(-2j/dh), positions 0..S (layers.py:52-60)
  {
    const int half = e->dh / 2, npos = e->S + 1;
    std::vector<float> ct((size_t)npos * half), st((size_t)npos * half);
    for (int j = 0; j < half; ++j) {
      const float expo = (float)(2 * j) / (float)e->dh;
      const float inv_freq = 1.0f / powf(cfg->rope_base, expo);
      for (int p = 0; p < npos; ++p) {
        const float ang = (float)p * inv_freq;
        ct[(size_t)p * half + j] = cosf(ang);
        st[(size_t)p * half + j] = sinf(ang);
      }
    }
    TRY(dev_alloc(e, &e->cos_tab, ct.size())); TRY(dev_alloc(e, &e->sin_tab, st.size()));
    CU(cudaMemcpy(e->cos_tab, ct.data(), ct.size() * 4, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(e->sin_tab, st.data(), st.size() * 4, cudaMemcpyHostToDevice));
  }
  e->layers.resize(cfg->num_layers);
  for (auto& L : e->layers) {
    TRY(dev_alloc(e, &L.w_qkv_t, (size_t)e->QW * e->D));
    TRY(dev_alloc(e, &L.w_out_t, (size_t)e->D * e->HD));
    TRY(dev_alloc(e, &L.w_up_t, (size_t)e->F * e->D));
    TRY(dev_alloc(e, &L.w_down_t, (size_t)e->D * e->F));
    TRY(gemm_plan_create(&L.p_qkv, e->hbuf, L.w_qkv_t, M, e->QW, e->D, false, e->err));
    if (e->fused_norm) {
      TRY(dev_alloc(e, &L.w_qkv_f, (size_t)e->QW * e->D));
      TRY(dev_alloc(e, &L.w_up_f, (size_t)e->F * e->D));
      TRY(gemm_plan_create(&L.p_qkv_f, e->x, L.w_qkv_f, M, e->QW, e->D, false, e->err));
      TRY(gemm_plan_create(&L.p_up_f, e->x, L.w_up_f, M, e->F, e->D, false, e->err));
    }
    TRY(gemm_plan_create(&L.p_out, e->attn, L.w_out_t, M, e->D, e->HD, e->HD <= 1024 && !cfg->primer_norm, e->err));
    TRY(gemm_plan_create(&L.p_up, e->hbuf, L.w_up_t, M, e->F, e->D, false, e->err));
    TRY(gemm_plan_create(&L.p_down, e->ffn, L.w_down_t, M, e->D, e->F, false, e->err));
#ifdef PHX_DIAGNOSTICS
    if (getenv("PHX_GEMM_COUNTERS")) {   // diagnostics: MMA-issuer wait counters by role, summed over layers and forwards
      if (!e->gemm_counters) {
        CU(cudaMalloc(reinterpret_cast<void**>(&e->gemm_counters), 4 * 8 * sizeof(unsigned long long)));
        CU(cudaMemset(e->gemm_counters, 0, 4 * 8 * sizeof(unsigned long long)));
      }
      L.p_qkv.counters = L.p_qkv_f.counters = e->gemm_counters;
      L.p_out.counters = e->gemm_counters + 8;
      L.p_up.counters = L.p_up_f.counters = e->gemm_counters + 16;
      L.p_down.counters = e->gemm_counters + 24;
    }
#endif
  }
  if (e->V + e->NC > 0) TRY(dev_alloc(e, &e->unembed_t, (size_t)(e->V + e->NC) * e->D));
  // staging for the host entry point
  {
    const size_t B = cfg->max_batch;
    const size_t H = (size_t)cfg->item.num_hashes;   // raw ids (8 bytes each) or pre-hashed rows (4 bytes x H each)
    const size_t per_id = 8 > 4 * H ? 8 : 4 * H;
    e->in_stage_bytes = B * ((size_t)e->S * (2 * per_id + 4 + 4) + (size_t)e->C * 2 * per_id) + 2 * (B + 1) * 4 + 64;
    // the batch-prep form: user and IP rows, one byte per action flag, eight continuous values per history slot, a
    // surface per candidate; every array starts on a 16-byte boundary
    const size_t prep_bytes = B * (4 * (size_t)(cfg->user.num_hashes + cfg->ip.num_hashes) +
                                   (size_t)e->Sh * (8 * H + 4 + (size_t)cfg->num_action_types + 4 * PHX_PREP_CONTINUOUS) +
                                   (size_t)e->C * (8 * H + 4)) + 10 * 16;
    if (prep_bytes > e->in_stage_bytes) e->in_stage_bytes = prep_bytes;
    CU(cudaMalloc(&e->in_stage_dev, e->in_stage_bytes));
    CU(cudaMallocHost(&e->in_stage_host, e->in_stage_bytes));
    const size_t rows = B * (size_t)(e->C > 0 ? e->C : 1);
    TRY(dev_alloc(e, &e->lp_dev, rows * (e->V > 0 ? e->V : 1)));
    TRY(dev_alloc(e, &e->cont_dev, rows * (e->NC > 0 ? e->NC : 1)));
    TRY(dev_alloc(e, &e->score_dev, rows));
    CU(cudaMallocHost(reinterpret_cast<void**>(&e->lp_host), rows * (e->V > 0 ? e->V : 1) * 4));
    CU(cudaMallocHost(reinterpret_cast<void**>(&e->cont_host), rows * (e->NC > 0 ? e->NC : 1) * 4));
    CU(cudaMallocHost(reinterpret_cast<void**>(&e->score_host), rows * 8));
  }
  // the memsets above ran on the default stream; every later launch uses the engine's own non-blocking stream, which
  // does not order itself behind them
  CU(cudaDeviceSynchronize());
#undef TRY
#undef CU
  *out = e;
  return PHX_OK;
}

void phx_engine_destroy(phx_engine* e) {
  if (!e) return;
  cudaSetDevice(e->device);
  if (e->stream) cudaStreamSynchronize(e->stream);
  for (auto p : e->ipc_opened) if (p) cudaIpcCloseMemHandle(p);
  auto fr = [](void* p) { if (p) cudaFree(p); };
  fr(e->gemm_counters);
  if (e->graph_exec) cudaGraphExecDestroy(e->graph_exec);
  for (auto& sl : e->slots) {
    fr(sl.in_dev); fr(sl.lp_dev); fr(sl.cont_dev); fr(sl.score_dev);
    if (sl.in_host) cudaFreeHost(sl.in_host);
    if (sl.lp_host) cudaFreeHost(sl.lp_host);
    if (sl.cont_host) cudaFreeHost(sl.cont_host);
    if (sl.score_host) cudaFreeHost(sl.score_host);
    if (sl.in_ready) cudaEventDestroy(sl.in_ready);
    if (sl.fwd_done) cudaEventDestroy(sl.fwd_done);
    if (sl.out_done) cudaEventDestroy(sl.out_done);
    for (auto& ev : sl.chunk) if (ev) cudaEventDestroy(ev);
  }
  if (e->copy_stream) cudaStreamDestroy(e->copy_stream);
  fr(e->table); fr(e->action_table); fr(e->surface_table); fr(e->final_norm); fr(e->unembed_t);
  for (auto& L : e->layers) {
    fr(L.pre_attn_norm); fr(L.pre_ffn_norm); fr(L.post_attn_norm); fr(L.post_ffn_norm); fr(L.q_norm); fr(L.k_norm);
    fr(L.w_qkv_t); fr(L.w_out_t); fr(L.w_up_t); fr(L.w_down_t); fr(L.w_qkv_f); fr(L.w_up_f);
  }
  fr(e->cos_tab); fr(e->sin_tab); fr(e->x); fr(e->hbuf); fr(e->qkv); fr(e->attn); fr(e->ffn); fr(e->tmp); fr(e->tokens);
  for (phx_engine::PackState* ps : {&e->pack_full, &e->pack_ragged}) { fr(ps->hist_off); fr(ps->cand_off); fr(ps->pos_rows); fr(ps->out_index); }
  fr(e->proj_hist_t); fr(e->proj_cand_t); fr(e->cat_hist); fr(e->cat_cand); fr(e->tok_proj); fr(e->proj_user_t); fr(e->cat_user);
  for (int i = 0; i < PHX_MAX_HIST_CONT; ++i) { fr(e->cont_w1[i]); fr(e->cont_w2[i]); }
  fr(e->x32); fr(e->h32); fr(e->qkv32); fr(e->attn32); fr(e->ffn32); fr(e->tmp32); fr(e->hist32);
  fr(e->x_alt); fr(e->seg_alt); fr(e->rowss_a_alt); fr(e->rowss_a); fr(e->rowss_f); fr(e->seg); fr(e->hashes); fr(e->err_flag); fr(e->in_stage_dev); fr(e->lp_dev); fr(e->cont_dev); fr(e->score_dev);
  if (e->in_stage_host) cudaFreeHost(e->in_stage_host);
  if (e->lp_host) cudaFreeHost(e->lp_host);
  if (e->cont_host) cudaFreeHost(e->cont_host);
  if (e->score_host) cudaFreeHost(e->score_host);
  if (e->ev0) cudaEventDestroy(e->ev0);
  if (e->ev1) cudaEventDestroy(e->ev1);
  for (auto& pe : e->prof_events) { cudaEventDestroy(pe.second.first); cudaEventDestroy(pe.second.second); }
  for (auto m : e->marks) if (m) cudaEventDestroy(m);
  if (e->ev_prefetch) cudaEventDestroy(e->ev_prefetch);
  for (auto d : e->ev_done) if (d) cudaEventDestroy(d);
  if (e->side_stream) cudaStreamDestroy(e->side_stream);
  if (e->stream) cudaStreamDestroy(e->stream);
  delete e;
}

phx_status phx_load_param(phx_engine* e, const char* name, const float* host, int64_t rows, int64_t cols) {
  if (e) { e->graph_key_valid = false; if (e->graph_exec) { cudaGraphExecDestroy(e->graph_exec); e->graph_exec = nullptr; } }   // a captured forward holds the old state
  if (!e || !name || !host) return PHX_E_ARG;
  cudaSetDevice(e->device);
  const std::string n(name);
  auto shape = [&](int64_t r, int64_t c) {
    if (rows == r && cols == c) return true;
    e->err = "phx_load_param(" + n + "): expected [" + std::to_string(r) + "," + std::to_string(c) + "], got [" +
             std::to_string(rows) + "," + std::to_string(cols) + "]";
    return false;
  };
  phx_status s = PHX_E_ARG;
  if (n == "action_table") { if (!shape(e->cfg.action_multi_hot ? 1 : e->cfg.num_action_types + 1, e->D)) return PHX_E_ARG; s = upload_bf16(e, &e->action_table, host, rows, cols, false); }
  else if (n == "surface_table") { if (!shape(e->cfg.num_surfaces + 1, e->D)) return PHX_E_ARG; s = upload_bf16(e, &e->surface_table, host, rows, cols, false); }
  else if (n == "final_norm") { if (!shape(1, e->D)) return PHX_E_ARG; s = upload_f32(e, &e->final_norm, host, e->D, true); }
  else if (n == "proj_hist" || n == "proj_cand") {
    if (!e->project) { e->err = "phx_load_param(" + n + "): the engine was created without token_project"; return PHX_E_ARG; }
    const bool h = n == "proj_hist";
    if (!shape(h ? e->Kh : e->Kc, e->D)) return PHX_E_ARG;
    s = upload_bf16(e, h ? &e->proj_hist_t : &e->proj_cand_t, host, rows, cols, true);
  }
  else if (n == "proj_user") {
    if (!e->project || !e->P) { e->err = "phx_load_param(proj_user): the engine was created without token_project and user_prefix"; return PHX_E_ARG; }
    if (!shape(e->Ku, e->D)) return PHX_E_ARG;
    s = upload_bf16(e, &e->proj_user_t, host, rows, cols, true);
  }
  else if (n.rfind("hist_cont", 0) == 0) {
    const size_t dot = n.find('.');
    const int i = dot == std::string::npos ? -1 : atoi(n.substr(9, dot - 9).c_str());
    const std::string f = dot == std::string::npos ? "" : n.substr(dot + 1);
    if (i < 0 || i >= e->cfg.num_hist_continuous || (f != "proj1" && f != "proj2")) { e->err = "unknown parameter " + n; return PHX_E_ARG; }
    if (f == "proj1") { if (!shape(1, e->cfg.hist_cont_hidden)) return PHX_E_ARG; s = upload_bf16(e, &e->cont_w1[i], host, rows, cols, false); }
    else { if (!shape(e->cfg.hist_cont_hidden, e->D)) return PHX_E_ARG; s = upload_bf16(e, &e->cont_w2[i], host, rows, cols, false); }
  }
  else if (n == "unembed" || n == "cont_unembed") {
    const bool cont = n == "cont_unembed";
    const int nout = cont ? e->NC : e->V;
    if (!shape(e->D, nout)) return PHX_E_ARG;
    std::vector<uint16_t> tmp((size_t)nout * e->D);
    for (int r = 0; r < e->D; ++r) for (int c = 0; c < nout; ++c) tmp[(size_t)c * e->D + r] = f32_to_bf16_bits(host[(size_t)r * nout + c]);
    cudaError_t ce = cudaMemcpy(e->unembed_t + (size_t)(cont ? e->V : 0) * e->D, tmp.data(), tmp.size() * 2, cudaMemcpyHostToDevice);
    if (ce != cudaSuccess) { e->err = cudaGetErrorString(ce); return PHX_E_CUDA; }
    s = PHX_OK;
  } else if (n.rfind("layer", 0) == 0) {
    const size_t dot = n.find('.');
    if (dot == std::string::npos) { e->err = "unknown parameter " + n; return PHX_E_ARG; }
    const int l = atoi(n.substr(5, dot - 5).c_str());
    if (l < 0 || l >= (int)e->layers.size()) { e->err = "layer index out of range: " + n; return PHX_E_ARG; }
    Layer& L = e->layers[l];
    const std::string f = n.substr(dot + 1);
    if (f == "pre_attn_norm") { if (!shape(1, e->D)) return PHX_E_ARG; s = upload_f32(e, &L.pre_attn_norm, host, e->D, true); }
    else if (f == "pre_ffn_norm") { if (!shape(1, e->D)) return PHX_E_ARG; s = upload_f32(e, &L.pre_ffn_norm, host, e->D, true); }
    else if (f == "post_attn_norm") { if (!shape(1, e->D)) return PHX_E_ARG; s = upload_f32(e, &L.post_attn_norm, host, e->D, true); }
    else if (f == "post_ffn_norm") { if (!shape(1, e->D)) return PHX_E_ARG; s = upload_f32(e, &L.post_ffn_norm, host, e->D, true); }
    else if (f == "q_norm") { if (!shape(1, e->HD)) return PHX_E_ARG; s = upload_f32(e, &L.q_norm, host, e->HD, true); }
    else if (f == "k_norm") { if (!shape(1, e->Hkv * e->dh)) return PHX_E_ARG; s = upload_f32(e, &L.k_norm, host, e->Hkv * e->dh, true); }
    else if (f == "w_qkv") { if (!shape(e->D, e->QW)) return PHX_E_ARG; s = upload_bf16(e, &L.w_qkv_t, host, rows, cols, true); }
    else if (f == "w_out") { if (!shape(e->HD, e->D)) return PHX_E_ARG; s = upload_bf16(e, &L.w_out_t, host, rows, cols, true); }
    else if (f == "w_up") { if (!shape(e->D, e->F)) return PHX_E_ARG; s = upload_bf16(e, &L.w_up_t, host, rows, cols, true); }
    else if (f == "w_down") { if (!shape(e->F, e->D)) return PHX_E_ARG; s = upload_bf16(e, &L.w_down_t, host, rows, cols, true); }
    else { e->err = "unknown parameter " + n; return PHX_E_ARG; }
  } else { e->err = "unknown parameter " + n; return PHX_E_ARG; }
  if (s == PHX_OK) { e->loaded[n] = true; e->folded_dirty = true; }
  return s;
}

phx_status phx_table_upload(phx_engine* e, int64_t row0, int64_t nrows, const uint16_t* host_bf16) {
  if (!e || !host_bf16 || row0 < 0 || nrows < 0 || row0 + nrows > e->table_rows) { if (e) e->err = "phx_table_upload: range"; return PHX_E_ARG; }
  const long long lo = (long long)e->table_rank * e->shard_rows;
  if (row0 < lo || row0 + nrows > lo + e->shard_rows) { e->err = "phx_table_upload: rows outside this engine's shard"; return PHX_E_ARG; }
  cudaSetDevice(e->device);
  PHX_CUDA_TRY(cudaMemcpy(e->table + (row0 - lo) * e->D, host_bf16, (size_t)nrows * e->D * 2, cudaMemcpyHostToDevice), e->err);
  return PHX_OK;
}

phx_status phx_table_fill_synthetic(phx_engine* e, uint32_t seed, float amp) {
  if (!e) return PHX_E_ARG;
  cudaSetDevice(e->device);
  const long long lo = (long long)e->table_rank * e->shard_rows;
  long long mine = e->table_rows - lo;
  if (mine > e->shard_rows) mine = e->shard_rows;
  if (mine < 0) mine = 0;
  phx_status s = table_fill_launch(e->table, lo, mine, e->D, seed, amp, e->stream, e->err);
  if (s) return s;
  PHX_CUDA_TRY(cudaStreamSynchronize(e->stream), e->err);
  return PHX_OK;
}

phx_status phx_table_ipc_handle(phx_engine* e, uint8_t out[PHX_IPC_HANDLE_BYTES]) {
  if (!e || !out) return PHX_E_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == PHX_IPC_HANDLE_BYTES, "IPC handle size");
  cudaSetDevice(e->device);
  cudaIpcMemHandle_t h;
  PHX_CUDA_TRY(cudaIpcGetMemHandle(&h, e->table), e->err);
  memcpy(out, &h, sizeof(h));
  return PHX_OK;
}

phx_status phx_table_attach_peer(phx_engine* e, int32_t rank, const uint8_t handle[PHX_IPC_HANDLE_BYTES]) {
  if (!e || !handle || rank < 0 || rank >= e->table_world || rank == e->table_rank) { if (e) e->err = "phx_table_attach_peer: bad rank"; return PHX_E_ARG; }
  cudaSetDevice(e->device);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  PHX_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), e->err);
  e->ipc_opened[rank] = p;
  e->shard_ptr[rank] = static_cast<const bf16*>(p);
  return PHX_OK;
}

phx_status phx_table_local_ptr(phx_engine* e, void** out) {
  if (!e || !out) return PHX_E_ARG;
  *out = e->table;
  return PHX_OK;
}

phx_status phx_table_attach_peer_ptr(phx_engine* e, int32_t rank, const void* shard_dev) {
  if (!e || !shard_dev || rank < 0 || rank >= e->table_world || rank == e->table_rank) { if (e) e->err = "phx_table_attach_peer_ptr: bad rank"; return PHX_E_ARG; }
  e->shard_ptr[rank] = static_cast<const bf16*>(shard_dev);
  return PHX_OK;
}

phx_status phx_set_blend(phx_engine* e, const phx_blend_spec* spec) {
  if (e) { e->graph_key_valid = false; if (e->graph_exec) { cudaGraphExecDestroy(e->graph_exec); e->graph_exec = nullptr; } }   // a captured forward holds the old state
  if (!e || !spec || spec->num_terms < 0 || spec->num_terms > PHX_MAX_BLEND_TERMS) { if (e) e->err = "phx_set_blend: bad spec"; return PHX_E_ARG; }
  for (int i = 0; i < spec->num_terms; ++i)
    if (spec->src[i] < 0 || spec->src[i] >= e->V + e->NC) { e->err = "phx_set_blend: term source out of range"; return PHX_E_ARG; }
  e->blend = *spec; e->has_blend = true;
  return PHX_OK;
}

namespace {
// the launches of one forward, in order, on the engine's stream
phx_status enqueue_forward(phx_engine* e, const phx_rank_batch* bd, const phx_rank_out* od, int B, bool tokens_ready,
                           const bf16* landing = nullptr, const int* pos = nullptr, const HashedIn* hb = nullptr) {
  phx_status s;
  phx_engine::PackState* pk = e->cur_pack;
  if (pk && (pk->ragged || pk->planned_batch != B)) {
    // positions of the packed rows and the output slot of every candidate row (the full plan only when B changed)
    if (!pk->ragged) { pk->Mh = (long long)B * e->S; pk->M = (long long)B * e->T; }
    e->last_launches++;
    if ((s = pack_plan_launch(pack_map(pk), B, e->S, e->C, pk->pos_rows, pk->out_index, e->stream, e->err))) return s;
    pk->planned_batch = pk->ragged ? -1 : B;
  }
  if (!tokens_ready && (s = build_tokens(e, bd, B, e->C, nullptr, nullptr, nullptr, nullptr, nullptr, landing, pos, hb))) return s;
  if ((s = run_trunk(e, B, e->T, e->S, e->S, e->split, e->n_tail))) return s;
  const bool f32 = e->fp32;
  HeadsArgs ha;
  ha.x = e->x; ha.final_gain = e->final_norm; ha.unembed_t = e->unembed_t;
  ha.B = B; ha.T = e->T; ha.S = e->S; ha.C = e->C; ha.D = e->D; ha.V = e->V; ha.NC = e->NC;
  if (e->split) { ha.x = e->x + (long long)B * e->S * e->D; ha.T = e->C; ha.S = 0; }   // the candidate block of the split layout
  if (pk) {   // packed rows: candidate rows back to back, scattered to their output slots; padded slots read zero
    ha.x = e->x + pk->Mh * e->D; ha.out_index = pk->out_index; ha.rows = pk->M - pk->Mh;
    if (pk->ragged) {
      const size_t rows = (size_t)B * e->C;
      if (od->log_probs) PHX_CUDA_TRY(cudaMemsetAsync(od->log_probs, 0, rows * e->V * 4, e->stream), e->err);
      if (od->continuous) PHX_CUDA_TRY(cudaMemsetAsync(od->continuous, 0, rows * e->NC * 4, e->stream), e->err);
      if (od->scores) PHX_CUDA_TRY(cudaMemsetAsync(od->scores, 0, rows * 8, e->stream), e->err);
    }
  }
  ha.eps = e->cfg.rms_eps; ha.output_scale = 2.0f * sqrtf(512.0f / (float)e->D);  // scaling.py:43-44
  ha.final_logit_cap = e->cfg.final_logit_cap; ha.dwell_norm_scale = e->cfg.dwell_norm_scale;
  ha.has_blend = e->has_blend ? 1 : 0;
  if (e->has_blend) ha.blend = e->blend; else memset(&ha.blend, 0, sizeof(ha.blend));
  ha.log_probs = od->log_probs; ha.continuous = od->continuous; ha.scores = od->scores;
  { ProfScope ps(e, KC_HEADS); if ((s = f32 ? f32_heads_launch(e->x32, ha, e->stream, e->err) : heads_launch(ha, e->stream, e->err))) return s; }
  e->last_launches++;
  return PHX_OK;
}
}  // namespace

namespace {
// the six input arrays of an id batch: a null one would be dereferenced on the device (a fault on a shared GPU)
bool batch_arrays_present(phx_engine* e, const phx_rank_batch* b, bool need_candidates, const char* who) {
  if (e->prep_extras) {
    e->err = std::string(who) + ": the engine is configured for batch-prep buffers (user_prefix / cand_surface / continuous history "
             "actions): use phx_rank_forward_prep";
    return false;
  }
  if (b->batch <= 0) return true;   // nothing is read
  if (b->hist_post_ids && b->hist_author_ids && b->hist_actions && b->hist_surfaces &&
      (!need_candidates || (b->cand_post_ids && b->cand_author_ids))) return true;
  e->err = std::string(who) + ": null input array";
  return false;
}
}  // namespace

phx_status phx_rank_forward_device(phx_engine* e, const phx_rank_batch* bd, const phx_rank_out* od) {
  if (!e) return PHX_E_ARG;
  // the plan a host-buffer call prepared for this forward is taken here, before anything can fail: it never outlives
  // the call it was made for
  phx_engine::PackState* const planned = e->pack_next;
  e->pack_next = nullptr;
  if (!bd || !od) return PHX_E_ARG;
  if (e->C <= 0) { e->err = "engine was created without candidates"; return PHX_E_ARG; }
  if (!batch_arrays_present(e, bd, true, "phx_rank_forward_device")) return PHX_E_ARG;
  if (bd->batch < 0 || bd->batch > e->cfg.max_batch) { e->err = "batch exceeds max_batch"; return PHX_E_CAPACITY; }
  if (!params_complete(e, true) || !shards_complete(e)) return PHX_E_STATE;
  cudaSetDevice(e->device);
  const int B = bd->batch;
  e->last_batch = B; e->last_launches = 0; e->prof_used = 0;
  e->cur_pack = e->pack ? (planned ? planned : &e->pack_full) : nullptr;
  if (B == 0) return PHX_OK;
  PHX_CUDA_TRY(cudaEventRecord(e->ev0, e->stream), e->err);
  phx_status s;
  if ((s = refresh_folded(e))) return s;
  bool tokens_ready = false;
  if (e->prefetch_valid && memcmp(&e->prefetch_key, bd, sizeof(*bd)) == 0) {
    // tokens of this batch were built ahead of time: adopt the alternate buffers
    PHX_CUDA_TRY(cudaStreamWaitEvent(e->stream, e->ev_prefetch, 0), e->err);
    std::swap(e->x, e->x_alt);
    std::swap(e->seg, e->seg_alt);
    std::swap(e->rowss_a, e->rowss_a_alt);
    tokens_ready = true;
  }
  e->prefetch_valid = false;
  // Graph replay: same batch size and the same buffers as the previous call (a serving loop over its own staging
  // buffers).  The first such repeat is captured; diagnostics, prefetching and buffer swaps keep the eager path.
  const bool same_key = e->graph_key_valid && memcmp(&e->graph_key_b, bd, sizeof(*bd)) == 0 && memcmp(&e->graph_key_o, od, sizeof(*od)) == 0;
  const bool eligible = e->graphs_enabled && !e->profile && !e->sync_debug && !e->debug_taps && !e->side_stream && !tokens_ready &&
                        !(e->cur_pack && e->cur_pack->ragged);   // a ragged plan changes the launches from call to call
  if (!same_key && e->graph_exec) { cudaGraphExecDestroy(e->graph_exec); e->graph_exec = nullptr; }
  if (eligible && same_key && e->graph_exec) {
    PHX_CUDA_TRY(cudaGraphLaunch(e->graph_exec, e->stream), e->err);
    e->last_launches = e->graph_launches;
  } else if (eligible && same_key) {
    bool captured = false;
    if (cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
      s = enqueue_forward(e, bd, od, B, false);
      cudaGraph_t g = nullptr;
      const cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
      if (s == PHX_OK && ce == cudaSuccess && g && cudaGraphInstantiate(&e->graph_exec, g, 0) == cudaSuccess) captured = true;
      if (g) cudaGraphDestroy(g);
    }
    if (captured) {
      e->graph_launches = e->last_launches;
      PHX_CUDA_TRY(cudaGraphLaunch(e->graph_exec, e->stream), e->err);
    } else {   // capture is an optimisation: fall back to plain launches for the rest of the engine's life
      cudaGetLastError();
      e->graph_exec = nullptr;
      e->graphs_enabled = false;
      e->last_launches = 0;
      if ((s = enqueue_forward(e, bd, od, B, false))) return s;
    }
  } else {
    if ((s = enqueue_forward(e, bd, od, B, tokens_ready))) return s;
  }
  e->graph_key_b = *bd; e->graph_key_o = *od; e->graph_key_valid = true;
  PHX_CUDA_TRY(cudaEventRecord(e->ev1, e->stream), e->err);
  if (e->ev_done[0]) { e->done_idx ^= 1; PHX_CUDA_TRY(cudaEventRecord(e->ev_done[e->done_idx], e->stream), e->err); }
  return PHX_OK;
}

namespace {
// Packed rows: the leading non-padding slots of every request (id 0 = padding) as exclusive prefix sums ho / co with
// B + 1 entries.  A batch with padding in front of a valid slot is planned over all its slots.  A request keeps at
// least one history row (a padded one when it has none), so every request has a key block.
void plan_ragged(const phx_rank_batch* bh, size_t B, size_t S, size_t C, int* ho, int* co) {
  bool front_filled = true;
  ho[0] = co[0] = 0;
  for (size_t b = 0; b < B && front_filled; ++b) {
    const int64_t* hpid = bh->hist_post_ids + b * S;
    const int64_t* cpid = bh->cand_post_ids + b * C;
    size_t hc = 0, cc = 0;
    while (hc < S && hpid[hc] != 0) ++hc;
    while (cc < C && cpid[cc] != 0) ++cc;
    for (size_t t = hc; t < S; ++t) if (hpid[t] != 0) front_filled = false;
    for (size_t c = cc; c < C; ++c) if (cpid[c] != 0) front_filled = false;
    ho[b + 1] = ho[b] + (int)(hc > 0 ? hc : 1);
    co[b + 1] = co[b] + (int)cc;
  }
  if (!front_filled)
    for (size_t b = 0; b < B; ++b) { ho[b + 1] = (int)((b + 1) * S); co[b + 1] = (int)((b + 1) * C); }
}

}  // namespace

phx_status phx_plan_ragged(const int64_t* hist_post_ids, const int64_t* cand_post_ids, int32_t B, int32_t S, int32_t C,
                           int32_t* hist_off, int32_t* cand_off) {
  if (!hist_post_ids || !cand_post_ids || !hist_off || !cand_off || B < 0 || S <= 0 || C <= 0) {
    set_global_error("phx_plan_ragged: bad argument");
    return PHX_E_ARG;
  }
  phx_rank_batch b;
  memset(&b, 0, sizeof(b));
  b.batch = B; b.hist_post_ids = hist_post_ids; b.cand_post_ids = cand_post_ids;
  plan_ragged(&b, (size_t)B, (size_t)S, (size_t)C, hist_off, cand_off);
  return PHX_OK;
}

phx_status phx_rank_forward_packed_device(phx_engine* e, const phx_rank_batch* bd, const int32_t* hist_off_dev,
                                          const int32_t* cand_off_dev, int64_t hist_rows, int64_t cand_rows,
                                          const phx_rank_out* od) {
  if (!e || !bd || !od || !hist_off_dev || !cand_off_dev) return PHX_E_ARG;
  if (!e->pack) { e->err = "phx_rank_forward_packed_device: the engine was created without pack_ragged"; return PHX_E_ARG; }
  const long long B = bd->batch;
  if (B <= 0 || B > e->cfg.max_batch) { e->err = "batch must be 1..max_batch"; return PHX_E_CAPACITY; }
  if (hist_rows < B || hist_rows > B * e->S || cand_rows < 0 || cand_rows > B * e->C) {
    e->err = "phx_rank_forward_packed_device: row totals do not fit the batch (every request keeps at least one history row)";
    return PHX_E_ARG;
  }
  phx_engine::PackState& pk = e->pack_device;
  pk.hist_off_view = hist_off_dev; pk.cand_off_view = cand_off_dev;
  pk.pos_rows = e->pack_ragged.pos_rows; pk.out_index = e->pack_ragged.out_index;
  pk.Mh = hist_rows; pk.M = hist_rows + cand_rows;
  pk.ragged = true;
  e->pack_next = &pk;
  return phx_rank_forward_device(e, bd, od);
}

// Row-sharded table with the exchange done by the host side (parallel.ShardedRanker): first the unified-table rows
// of every token slot, then, once their rows sit in a landing buffer, the forward from there.
phx_status phx_rank_rows_device(phx_engine* e, const phx_rank_batch* bd, int32_t* rows_dev, void* stream) {
  if (!e || !bd || !rows_dev) return PHX_E_ARG;
  if (e->C <= 0) { e->err = "engine was created without candidates"; return PHX_E_ARG; }
  if (!batch_arrays_present(e, bd, true, "phx_rank_rows_device")) return PHX_E_ARG;
  if (bd->batch <= 0 || bd->batch > e->cfg.max_batch) { e->err = "batch must be 1..max_batch"; return PHX_E_CAPACITY; }
  cudaSetDevice(e->device);
  return build_tokens(e, bd, bd->batch, e->C, nullptr, nullptr, stream ? (cudaStream_t)stream : e->stream, nullptr, rows_dev);
}

phx_status phx_rank_forward_rows_device(phx_engine* e, const phx_rank_batch* bd, const uint16_t* landing_dev, const int32_t* pos_dev,
                                        const phx_rank_out* od) {
  if (!e || !bd || !od || !landing_dev || !pos_dev) return PHX_E_ARG;
  if (e->C <= 0) { e->err = "engine was created without candidates"; return PHX_E_ARG; }
  if (!batch_arrays_present(e, bd, true, "phx_rank_forward_rows_device")) return PHX_E_ARG;
  if (bd->batch <= 0 || bd->batch > e->cfg.max_batch) { e->err = "batch must be 1..max_batch"; return PHX_E_CAPACITY; }
  if (!params_complete(e, true)) return PHX_E_STATE;
  cudaSetDevice(e->device);
  const int B = bd->batch;
  e->last_batch = B; e->last_launches = 0; e->prof_used = 0;
  e->prefetch_valid = false;
  e->graph_key_valid = false;
  e->cur_pack = e->pack ? &e->pack_full : nullptr;
  PHX_CUDA_TRY(cudaEventRecord(e->ev0, e->stream), e->err);
  phx_status s;
  if ((s = refresh_folded(e))) return s;
  if ((s = enqueue_forward(e, bd, od, B, false, (const bf16*)landing_dev, pos_dev))) return s;
  PHX_CUDA_TRY(cudaEventRecord(e->ev1, e->stream), e->err);
  if (e->ev_done[0]) { e->done_idx ^= 1; PHX_CUDA_TRY(cudaEventRecord(e->ev_done[e->done_idx], e->stream), e->err); }
  return PHX_OK;
}

namespace {
// One forward from pre-hashed rows, asynchronous on the engine's stream.
phx_status forward_hashed_core(phx_engine* e, const HashedIn& in, int B, const phx_rank_out* od) {
  if (!params_complete(e, true) || !shards_complete(e)) return PHX_E_STATE;
  cudaSetDevice(e->device);
  e->last_batch = B; e->last_launches = 0; e->prof_used = 0;
  e->prefetch_valid = false;
  e->graph_key_valid = false;   // plain launches: the graph cache is keyed on id batches
  e->cur_pack = e->pack ? &e->pack_full : nullptr;
  if (B == 0) return PHX_OK;
  PHX_CUDA_TRY(cudaEventRecord(e->ev0, e->stream), e->err);
  phx_status s;
  if ((s = refresh_folded(e))) return s;
  if ((s = enqueue_forward(e, nullptr, od, B, false, nullptr, nullptr, &in))) return s;
  PHX_CUDA_TRY(cudaEventRecord(e->ev1, e->stream), e->err);
  if (e->ev_done[0]) { e->done_idx ^= 1; PHX_CUDA_TRY(cudaEventRecord(e->ev_done[e->done_idx], e->stream), e->err); }
  return PHX_OK;
}

// results of the forward that was just enqueued: device -> pinned -> the caller's arrays; waits for the stream
phx_status fetch_outputs(phx_engine* e, size_t B, const phx_rank_out* oh) {
  const size_t rows = B * e->C;
  if (oh->log_probs) PHX_CUDA_TRY(cudaMemcpyAsync(e->lp_host, e->lp_dev, rows * e->V * 4, cudaMemcpyDeviceToHost, e->stream), e->err);
  if (oh->continuous) PHX_CUDA_TRY(cudaMemcpyAsync(e->cont_host, e->cont_dev, rows * e->NC * 4, cudaMemcpyDeviceToHost, e->stream), e->err);
  if (oh->scores && e->has_blend) PHX_CUDA_TRY(cudaMemcpyAsync(e->score_host, e->score_dev, rows * 8, cudaMemcpyDeviceToHost, e->stream), e->err);
  PHX_CUDA_TRY(cudaStreamSynchronize(e->stream), e->err);
  if (oh->log_probs) memcpy(oh->log_probs, e->lp_host, rows * e->V * 4);
  if (oh->continuous) memcpy(oh->continuous, e->cont_host, rows * e->NC * 4);
  if (oh->scores && e->has_blend) memcpy(oh->scores, e->score_host, rows * 8);
  return check_err_flag(e);
}

bool hashed_arrays_present(phx_engine* e, const phx_rank_batch_hashed* b, const char* who) {
  if (e->prep_extras) {
    e->err = std::string(who) + ": the engine is configured for batch-prep buffers (user_prefix / cand_surface / continuous history "
             "actions): use phx_rank_forward_prep";
    return false;
  }
  if (b->batch <= 0) return true;
  if (b->hist_post_hashes && b->hist_author_hashes && b->cand_post_hashes && b->cand_author_hashes && b->hist_actions && b->hist_surfaces)
    return true;
  e->err = std::string(who) + ": null input array";
  return false;
}

// the buffers the configuration reads must be there; the others are ignored
bool prep_arrays_present(phx_engine* e, const phx_rank_batch_prep* b, const char* who) {
  if (!e->cfg.action_multi_hot) { e->err = std::string(who) + ": history_actions is a set per position: the engine needs action_multi_hot = 1"; return false; }
  if (b->batch <= 0) return true;
  const bool ok = b->history_post_hashes && b->history_auth_hashes && b->history_product_surfaces && b->history_actions &&
                  b->candidate_post_hashes && b->candidate_auth_hashes && (!e->P || b->user_hashes) &&
                  (!e->cfg.cand_surface || b->candidate_product_surfaces) &&
                  (e->cfg.num_hist_continuous == 0 || b->history_continuous_actions);
  if (!ok) e->err = std::string(who) + ": null input array";
  return ok;
}

HashedIn hashed_in(const phx_rank_batch_prep* b) {
  HashedIn in;
  in.user_hashes = b->user_hashes; in.user_ip_hashes = b->user_ip_hashes;
  in.hist_post = b->history_post_hashes; in.hist_author = b->history_auth_hashes; in.hist_surfaces = b->history_product_surfaces;
  in.hist_actions_bool = b->history_actions; in.hist_cont = b->history_continuous_actions;
  in.cand_post = b->candidate_post_hashes; in.cand_author = b->candidate_auth_hashes; in.cand_surfaces = b->candidate_product_surfaces;
  return in;
}
}  // namespace

phx_status phx_rank_forward_hashed_device(phx_engine* e, const phx_rank_batch_hashed* hb, const phx_rank_out* od) {
  if (!e || !hb || !od) return PHX_E_ARG;
  if (e->C <= 0) { e->err = "engine was created without candidates"; return PHX_E_ARG; }
  if (hb->batch < 0 || hb->batch > e->cfg.max_batch) { e->err = "batch exceeds max_batch"; return PHX_E_CAPACITY; }
  if (!hashed_arrays_present(e, hb, "phx_rank_forward_hashed_device")) return PHX_E_ARG;
  HashedIn in;
  in.hist_post = hb->hist_post_hashes; in.hist_author = hb->hist_author_hashes; in.cand_post = hb->cand_post_hashes;
  in.cand_author = hb->cand_author_hashes; in.hist_actions = hb->hist_actions; in.hist_surfaces = hb->hist_surfaces;
  return forward_hashed_core(e, in, hb->batch, od);
}

phx_status phx_rank_forward_hashed(phx_engine* e, const phx_rank_batch_hashed* bh, const phx_rank_out* oh) {
  if (!e || !bh || !oh) return PHX_E_ARG;
  if (e->C <= 0) { e->err = "engine was created without candidates"; return PHX_E_ARG; }
  if (bh->batch < 0 || bh->batch > e->cfg.max_batch) { e->err = "batch exceeds max_batch"; return PHX_E_CAPACITY; }
  if (!hashed_arrays_present(e, bh, "phx_rank_forward_hashed")) return PHX_E_ARG;
  cudaSetDevice(e->device);
  const size_t B = bh->batch, S = e->S, C = e->C, H = e->cfg.item.num_hashes;
  if (B == 0) return PHX_OK;
  uint8_t* hp = (uint8_t*)e->in_stage_host;
  uint8_t* dp = (uint8_t*)e->in_stage_dev;
  size_t off = 0;
  phx_rank_batch_hashed bd; bd.batch = bh->batch; bd._pad = 0;
  auto put = [&](const void* src, size_t bytes) { memcpy(hp + off, src, bytes); const void* d = dp + off; off += bytes; return (const int32_t*)d; };
  bd.hist_post_hashes = put(bh->hist_post_hashes, B * S * H * 4);
  bd.hist_author_hashes = put(bh->hist_author_hashes, B * S * H * 4);
  bd.cand_post_hashes = put(bh->cand_post_hashes, B * C * H * 4);
  bd.cand_author_hashes = put(bh->cand_author_hashes, B * C * H * 4);
  bd.hist_actions = put(bh->hist_actions, B * S * 4);
  bd.hist_surfaces = put(bh->hist_surfaces, B * S * 4);
  PHX_CUDA_TRY(cudaMemcpyAsync(dp, hp, off, cudaMemcpyHostToDevice, e->stream), e->err);
  phx_rank_out od; od.log_probs = e->lp_dev; od.continuous = e->cont_dev; od.scores = e->score_dev;
  phx_status s = phx_rank_forward_hashed_device(e, &bd, &od);
  if (s) return s;
  return fetch_outputs(e, B, oh);
}

phx_status phx_rank_forward_prep_device(phx_engine* e, const phx_rank_batch_prep* pb, const phx_rank_out* od) {
  if (!e || !pb || !od) return PHX_E_ARG;
  if (e->C <= 0) { e->err = "engine was created without candidates"; return PHX_E_ARG; }
  if (pb->batch < 0 || pb->batch > e->cfg.max_batch) { e->err = "batch exceeds max_batch"; return PHX_E_CAPACITY; }
  if (!prep_arrays_present(e, pb, "phx_rank_forward_prep_device")) return PHX_E_ARG;
  return forward_hashed_core(e, hashed_in(pb), pb->batch, od);
}

phx_status phx_rank_forward_prep(phx_engine* e, const phx_rank_batch_prep* bh, const phx_rank_out* oh) {
  if (!e || !bh || !oh) return PHX_E_ARG;
  if (e->C <= 0) { e->err = "engine was created without candidates"; return PHX_E_ARG; }
  if (bh->batch < 0 || bh->batch > e->cfg.max_batch) { e->err = "batch exceeds max_batch"; return PHX_E_CAPACITY; }
  if (!prep_arrays_present(e, bh, "phx_rank_forward_prep")) return PHX_E_ARG;
  cudaSetDevice(e->device);
  const size_t B = bh->batch, S = e->Sh, C = e->C, H = e->cfg.item.num_hashes, V = e->cfg.num_action_types;
  const size_t Hu = e->cfg.user.num_hashes, Hip = e->cfg.ip.num_hashes;
  if (B == 0) return PHX_OK;
  uint8_t* hp = (uint8_t*)e->in_stage_host;
  uint8_t* dp = (uint8_t*)e->in_stage_dev;
  size_t off = 0;
  // only what the configuration reads is copied; every array starts on a 16-byte boundary of the staging block
  bool fits = true;
  auto put = [&](const void* src, size_t bytes, bool wanted) -> const void* {
    if (!wanted || !src) return nullptr;
    if (off + bytes > e->in_stage_bytes) { fits = false; return nullptr; }
    memcpy(hp + off, src, bytes);
    const void* d = dp + off;
    off = (off + bytes + 15) & ~(size_t)15;
    return d;
  };
  phx_rank_batch_prep bd; memset(&bd, 0, sizeof(bd)); bd.batch = bh->batch;
  bd.user_hashes = (const int32_t*)put(bh->user_hashes, B * Hu * 4, e->P != 0);
  bd.user_ip_hashes = (const int32_t*)put(bh->user_ip_hashes, B * Hip * 4, e->P != 0 && Hip > 0);
  bd.history_post_hashes = (const int32_t*)put(bh->history_post_hashes, B * S * H * 4, true);
  bd.history_auth_hashes = (const int32_t*)put(bh->history_auth_hashes, B * S * H * 4, true);
  bd.history_product_surfaces = (const int32_t*)put(bh->history_product_surfaces, B * S * 4, true);
  bd.history_actions = (const uint8_t*)put(bh->history_actions, B * S * V, true);
  bd.history_continuous_actions = (const float*)put(bh->history_continuous_actions, B * S * PHX_PREP_CONTINUOUS * 4, e->cfg.num_hist_continuous > 0);
  bd.candidate_post_hashes = (const int32_t*)put(bh->candidate_post_hashes, B * C * H * 4, true);
  bd.candidate_auth_hashes = (const int32_t*)put(bh->candidate_auth_hashes, B * C * H * 4, true);
  bd.candidate_product_surfaces = (const int32_t*)put(bh->candidate_product_surfaces, B * C * 4, e->cfg.cand_surface != 0);
  if (!fits) { e->err = "phx_rank_forward_prep: staging block too small"; return PHX_E_CAPACITY; }
  PHX_CUDA_TRY(cudaMemcpyAsync(dp, hp, off, cudaMemcpyHostToDevice, e->stream), e->err);
  phx_rank_out od; od.log_probs = e->lp_dev; od.continuous = e->cont_dev; od.scores = e->score_dev;
  phx_status s = phx_rank_forward_prep_device(e, &bd, &od);
  if (s) return s;
  return fetch_outputs(e, B, oh);
}

phx_status phx_rank_prefetch_device(phx_engine* e, const phx_rank_batch* bd) {
  if (!e || !bd) return PHX_E_ARG;
  if (e->C <= 0) { e->err = "engine was created without candidates"; return PHX_E_ARG; }
  if (!batch_arrays_present(e, bd, true, "phx_rank_prefetch_device")) return PHX_E_ARG;
  if (bd->batch <= 0 || bd->batch > e->cfg.max_batch) { e->err = "batch exceeds max_batch"; return PHX_E_CAPACITY; }
  if (e->fp32) { e->err = "token prefetch is not available on the full-precision path"; return PHX_E_ARG; }
  if (e->pack) { e->err = "token prefetch is not available on an engine that packs ragged batches"; return PHX_E_ARG; }
  if (!params_complete(e, true) || !shards_complete(e)) return PHX_E_STATE;
  cudaSetDevice(e->device);
  if (!e->side_stream) {
    PHX_CUDA_TRY(cudaStreamCreateWithFlags(&e->side_stream, cudaStreamNonBlocking), e->err);
    PHX_CUDA_TRY(cudaEventCreateWithFlags(&e->ev_prefetch, cudaEventDisableTiming), e->err);
    for (int i = 0; i < 2; ++i) PHX_CUDA_TRY(cudaEventCreateWithFlags(&e->ev_done[i], cudaEventDisableTiming), e->err);
    PHX_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&e->x_alt), (size_t)e->max_tokens * e->D * sizeof(bf16)), e->err);
    PHX_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&e->seg_alt), (size_t)e->max_tokens * sizeof(int)), e->err);
    PHX_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&e->rowss_a_alt), (size_t)e->max_tokens * (e->D / 64) * sizeof(float)), e->err);
    for (int i = 0; i < 2; ++i) PHX_CUDA_TRY(cudaEventRecord(e->ev_done[i], e->stream), e->err);
  }
  // Call order per step: forward(batch i), then prefetch(batch i+1).  The alternate buffers were the working
  // buffers of forward(i-1); the side stream waits for THAT forward's end (the event before the most recent one),
  // not for forward(i), so the gather overlaps forward(i).
  PHX_CUDA_TRY(cudaStreamWaitEvent(e->side_stream, e->ev_done[e->done_idx ^ 1], 0), e->err);
  phx_status s = build_tokens(e, bd, bd->batch, e->C, e->x_alt, e->seg_alt, e->side_stream, e->rowss_a_alt);
  if (s) return s;
  PHX_CUDA_TRY(cudaEventRecord(e->ev_prefetch, e->side_stream), e->err);
  e->prefetch_key = *bd;
  e->prefetch_valid = true;
  return PHX_OK;
}

phx_status phx_rank_forward(phx_engine* e, const phx_rank_batch* bh, const phx_rank_out* oh) {
  if (!e || !bh || !oh) return PHX_E_ARG;
  if (bh->batch < 0 || bh->batch > e->cfg.max_batch) { e->err = "batch exceeds max_batch"; return PHX_E_CAPACITY; }
  if (!batch_arrays_present(e, bh, true, "phx_rank_forward")) return PHX_E_ARG;
  cudaSetDevice(e->device);
  const size_t B = bh->batch, S = e->S, C = e->C;
  if (B == 0) return PHX_OK;
  // pack the six input arrays into one pinned block -> one H2D copy
  uint8_t* hp = (uint8_t*)e->in_stage_host;
  uint8_t* dp = (uint8_t*)e->in_stage_dev;
  size_t off = 0;
  phx_rank_batch bd; bd.batch = bh->batch; bd._pad = 0;
  auto put = [&](const void* src, size_t bytes) { memcpy(hp + off, src, bytes); const void* d = dp + off; off += bytes; return d; };
  bd.hist_post_ids = (const int64_t*)put(bh->hist_post_ids, B * S * 8);
  bd.hist_author_ids = (const int64_t*)put(bh->hist_author_ids, B * S * 8);
  bd.cand_post_ids = (const int64_t*)put(bh->cand_post_ids, B * C * 8);
  bd.cand_author_ids = (const int64_t*)put(bh->cand_author_ids, B * C * 8);
  bd.hist_actions = (const int32_t*)put(bh->hist_actions, B * S * 4);
  bd.hist_surfaces = (const int32_t*)put(bh->hist_surfaces, B * S * 4);
  if (e->pack) {
    int* ho = e->pack_host.data();
    int* co = ho + (B + 1);
    plan_ragged(bh, B, S, C, ho, co);
    off = (off + 15) & ~(size_t)15;
    phx_engine::PackState& pk = e->pack_ragged;
    pk.hist_off_view = (const int*)put(ho, (B + 1) * 4);   // the plan reads its offsets from the staged block
    pk.cand_off_view = (const int*)put(co, (B + 1) * 4);
    pk.Mh = ho[B]; pk.M = (long long)ho[B] + co[B];
    PHX_CUDA_TRY(cudaMemcpyAsync(dp, hp, off, cudaMemcpyHostToDevice, e->stream), e->err);
    e->pack_next = &pk;
  } else {
    PHX_CUDA_TRY(cudaMemcpyAsync(dp, hp, off, cudaMemcpyHostToDevice, e->stream), e->err);
  }
  phx_rank_out od; od.log_probs = e->lp_dev; od.continuous = e->cont_dev; od.scores = e->score_dev;
  phx_status s = phx_rank_forward_device(e, &bd, &od);
  if (s) return s;
  const size_t rows = B * C;
  // results come back in four row chunks: while the host copies chunk i out of the pinned staging block, chunk i+1
  // is still on the bus
  constexpr int NCH = 4;
  const size_t step = (rows + NCH - 1) / NCH;
  for (int i = 0; i < NCH; ++i) {
    const size_t r0 = i * step, r1 = (r0 + step < rows) ? r0 + step : rows;
    if (r0 < r1) {
      if (oh->log_probs) PHX_CUDA_TRY(cudaMemcpyAsync(e->lp_host + r0 * e->V, e->lp_dev + r0 * e->V, (r1 - r0) * e->V * 4, cudaMemcpyDeviceToHost, e->stream), e->err);
      if (oh->continuous) PHX_CUDA_TRY(cudaMemcpyAsync(e->cont_host + r0 * e->NC, e->cont_dev + r0 * e->NC, (r1 - r0) * e->NC * 4, cudaMemcpyDeviceToHost, e->stream), e->err);
      if (oh->scores && e->has_blend) PHX_CUDA_TRY(cudaMemcpyAsync(e->score_host + r0, e->score_dev + r0, (r1 - r0) * 8, cudaMemcpyDeviceToHost, e->stream), e->err);
    }
    if (!e->ev_chunk[i]) PHX_CUDA_TRY(cudaEventCreateWithFlags(&e->ev_chunk[i], cudaEventDisableTiming), e->err);
    PHX_CUDA_TRY(cudaEventRecord(e->ev_chunk[i], e->stream), e->err);
  }
  for (int i = 0; i < NCH; ++i) {
    PHX_CUDA_TRY(cudaEventSynchronize(e->ev_chunk[i]), e->err);
    const size_t r0 = i * step, r1 = (r0 + step < rows) ? r0 + step : rows;
    if (r0 >= r1) continue;
    if (oh->log_probs) memcpy(oh->log_probs + r0 * e->V, e->lp_host + r0 * e->V, (r1 - r0) * e->V * 4);
    if (oh->continuous) memcpy(oh->continuous + r0 * e->NC, e->cont_host + r0 * e->NC, (r1 - r0) * e->NC * 4);
    if (oh->scores && e->has_blend) memcpy(oh->scores + r0, e->score_host + r0, (r1 - r0) * 8);
  }
  PHX_CUDA_TRY(cudaStreamSynchronize(e->stream), e->err);
  return check_err_flag(e);
}

// ---- pipelined host-buffer requests ------------------------------------------------------------------------------
namespace {
phx_status slots_init(phx_engine* e) {
  if (e->copy_stream) return PHX_OK;
  PHX_CUDA_TRY(cudaStreamCreateWithFlags(&e->copy_stream, cudaStreamNonBlocking), e->err);
  const size_t rows = (size_t)e->cfg.max_batch * e->C;
  for (auto& sl : e->slots) {
    PHX_CUDA_TRY(cudaMalloc(&sl.in_dev, e->in_stage_bytes), e->err);
    PHX_CUDA_TRY(cudaMallocHost(&sl.in_host, e->in_stage_bytes), e->err);
    PHX_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&sl.lp_dev), rows * (e->V > 0 ? e->V : 1) * 4), e->err);
    PHX_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&sl.cont_dev), rows * (e->NC > 0 ? e->NC : 1) * 4), e->err);
    PHX_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&sl.score_dev), rows * 8), e->err);
    PHX_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&sl.lp_host), rows * (e->V > 0 ? e->V : 1) * 4), e->err);
    PHX_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&sl.cont_host), rows * (e->NC > 0 ? e->NC : 1) * 4), e->err);
    PHX_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&sl.score_host), rows * 8), e->err);
    PHX_CUDA_TRY(cudaEventCreateWithFlags(&sl.in_ready, cudaEventDisableTiming), e->err);
    PHX_CUDA_TRY(cudaEventCreateWithFlags(&sl.fwd_done, cudaEventDisableTiming), e->err);
    PHX_CUDA_TRY(cudaEventCreateWithFlags(&sl.out_done, cudaEventDisableTiming), e->err);
    for (auto& ev : sl.chunk) PHX_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), e->err);
  }
  return PHX_OK;
}
constexpr int SLOT_CHUNKS = 4;
}  // namespace

phx_status phx_rank_submit(phx_engine* e, const phx_rank_batch* bh, int32_t slot) {
  if (!e || !bh || slot < 0 || slot > 1) return PHX_E_ARG;
  if (bh->batch <= 0 || bh->batch > e->cfg.max_batch) { e->err = "batch must be 1..max_batch"; return PHX_E_CAPACITY; }
  if (!batch_arrays_present(e, bh, true, "phx_rank_submit")) return PHX_E_ARG;
  cudaSetDevice(e->device);
  phx_status s = slots_init(e);
  if (s) return s;
  auto& sl = e->slots[slot];
  if (sl.busy) { e->err = "phx_rank_submit: the slot holds a request that has not been collected"; return PHX_E_STATE; }
  const size_t B = bh->batch, S = e->S, C = e->C;
  uint8_t* hp = (uint8_t*)sl.in_host;
  uint8_t* dp = (uint8_t*)sl.in_dev;
  size_t off = 0;
  phx_rank_batch bd; bd.batch = bh->batch; bd._pad = 0;
  auto put = [&](const void* src, size_t bytes) { memcpy(hp + off, src, bytes); const void* d = dp + off; off += bytes; return d; };
  bd.hist_post_ids = (const int64_t*)put(bh->hist_post_ids, B * S * 8);
  bd.hist_author_ids = (const int64_t*)put(bh->hist_author_ids, B * S * 8);
  bd.cand_post_ids = (const int64_t*)put(bh->cand_post_ids, B * C * 8);
  bd.cand_author_ids = (const int64_t*)put(bh->cand_author_ids, B * C * 8);
  bd.hist_actions = (const int32_t*)put(bh->hist_actions, B * S * 4);
  bd.hist_surfaces = (const int32_t*)put(bh->hist_surfaces, B * S * 4);
  if (e->pack) {   // packed rows: this request's counts travel in the slot's block, its plan shares the engine's row arrays
    sl.pack_host.resize(2 * (B + 1));
    int* ho = sl.pack_host.data();
    int* co = ho + (B + 1);
    plan_ragged(bh, B, S, C, ho, co);
    off = (off + 15) & ~(size_t)15;
    sl.pack.hist_off_view = (const int*)put(ho, (B + 1) * 4);
    sl.pack.cand_off_view = (const int*)put(co, (B + 1) * 4);
    sl.pack.pos_rows = e->pack_ragged.pos_rows; sl.pack.out_index = e->pack_ragged.out_index;
    sl.pack.Mh = ho[B]; sl.pack.M = (long long)ho[B] + co[B];
    sl.pack.ragged = true;
    e->pack_next = &sl.pack;
  }
  // inputs: on the copy stream, once the forward that last read this slot's device block is done
  PHX_CUDA_TRY(cudaStreamWaitEvent(e->copy_stream, sl.fwd_done, 0), e->err);
  PHX_CUDA_TRY(cudaMemcpyAsync(dp, hp, off, cudaMemcpyHostToDevice, e->copy_stream), e->err);
  PHX_CUDA_TRY(cudaEventRecord(sl.in_ready, e->copy_stream), e->err);
  // forward: after the inputs have landed and the slot's previous results have left its device block
  PHX_CUDA_TRY(cudaStreamWaitEvent(e->stream, sl.in_ready, 0), e->err);
  PHX_CUDA_TRY(cudaStreamWaitEvent(e->stream, sl.out_done, 0), e->err);
  phx_rank_out od; od.log_probs = sl.lp_dev; od.continuous = sl.cont_dev; od.scores = sl.score_dev;
  if ((s = phx_rank_forward_device(e, &bd, &od))) return s;
  PHX_CUDA_TRY(cudaEventRecord(sl.fwd_done, e->stream), e->err);
  // results: back on the copy stream, in row chunks
  PHX_CUDA_TRY(cudaStreamWaitEvent(e->copy_stream, sl.fwd_done, 0), e->err);
  const size_t rows = B * C, step = (rows + SLOT_CHUNKS - 1) / SLOT_CHUNKS;
  for (int i = 0; i < SLOT_CHUNKS; ++i) {
    const size_t r0 = i * step, r1 = (r0 + step < rows) ? r0 + step : rows;
    if (r0 < r1) {
      PHX_CUDA_TRY(cudaMemcpyAsync(sl.lp_host + r0 * e->V, sl.lp_dev + r0 * e->V, (r1 - r0) * e->V * 4, cudaMemcpyDeviceToHost, e->copy_stream), e->err);
      PHX_CUDA_TRY(cudaMemcpyAsync(sl.cont_host + r0 * e->NC, sl.cont_dev + r0 * e->NC, (r1 - r0) * e->NC * 4, cudaMemcpyDeviceToHost, e->copy_stream), e->err);
      if (e->has_blend) PHX_CUDA_TRY(cudaMemcpyAsync(sl.score_host + r0, sl.score_dev + r0, (r1 - r0) * 8, cudaMemcpyDeviceToHost, e->copy_stream), e->err);
    }
    PHX_CUDA_TRY(cudaEventRecord(sl.chunk[i], e->copy_stream), e->err);
  }
  PHX_CUDA_TRY(cudaEventRecord(sl.out_done, e->copy_stream), e->err);
  sl.busy = true;
  sl.batch = bh->batch;
  return PHX_OK;
}

phx_status phx_rank_collect(phx_engine* e, int32_t slot, const phx_rank_out* oh) {
  if (!e || !oh || slot < 0 || slot > 1) return PHX_E_ARG;
  auto& sl = e->slots[slot];
  if (!sl.busy) { e->err = "phx_rank_collect: nothing was submitted to this slot"; return PHX_E_STATE; }
  cudaSetDevice(e->device);
  const size_t rows = (size_t)sl.batch * e->C, step = (rows + SLOT_CHUNKS - 1) / SLOT_CHUNKS;
  for (int i = 0; i < SLOT_CHUNKS; ++i) {
    PHX_CUDA_TRY(cudaEventSynchronize(sl.chunk[i]), e->err);
    const size_t r0 = i * step, r1 = (r0 + step < rows) ? r0 + step : rows;
    if (r0 >= r1) continue;
    if (oh->log_probs) memcpy(oh->log_probs + r0 * e->V, sl.lp_host + r0 * e->V, (r1 - r0) * e->V * 4);
    if (oh->continuous) memcpy(oh->continuous + r0 * e->NC, sl.cont_host + r0 * e->NC, (r1 - r0) * e->NC * 4);
    if (oh->scores && e->has_blend) memcpy(oh->scores + r0, sl.score_host + r0, (r1 - r0) * 8);
  }
  sl.busy = false;
  return check_err_flag(e);
}

phx_status phx_sync(phx_engine* e) {
  if (!e) return PHX_E_ARG;
  cudaSetDevice(e->device);
  PHX_CUDA_TRY(cudaStreamSynchronize(e->stream), e->err);
  return check_err_flag(e);
}

phx_status phx_set_wait_limit_us(phx_engine* e, uint32_t microseconds) {
  if (!e) return PHX_E_ARG;
  cudaSetDevice(e->device);
  PHX_CUDA_TRY(cudaStreamSynchronize(e->stream), e->err);
  const int v = (int)(microseconds > 0x7FFFFFFFu ? 0x7FFFFFFFu : microseconds);
  PHX_CUDA_TRY(cudaMemcpy(e->err_flag + 1, &v, sizeof(int), cudaMemcpyHostToDevice), e->err);
  return PHX_OK;
}

phx_status phx_wait_selftest(phx_engine* e) {
  if (!e) return PHX_E_ARG;
  cudaSetDevice(e->device);
  phx_status s = wait_selftest_launch(e->err_flag, e->stream, e->err);
  if (s) return s;
  return phx_sync(e);
}

int32_t phx_dispatch_counts(int64_t* out, int32_t n) {
  for (int i = 0; i < n && i < DK_COUNT; ++i) out[i] = g_dispatch[i].load(std::memory_order_relaxed);
  return DK_COUNT;
}

const char* phx_dispatch_name(int32_t kind) {
  static const char* names[DK_COUNT] = {"attn.strip", "attn.stream", "attn.tcgen05", "attn.resident", "gemm.pair256", "gemm.pair128",
                                        "gemm.cta256", "gemm.cta128", "gemm.simt", "scan.tcgen05", "scan.mma", "topk.exact", "attn.pingpong"};
  return (kind >= 0 && kind < DK_COUNT) ? names[kind] : "";
}

phx_status phx_last_device_ms(phx_engine* e, float* ms) {
  if (!e || !ms) return PHX_E_ARG;
  PHX_CUDA_TRY(cudaEventSynchronize(e->ev1), e->err);
  PHX_CUDA_TRY(cudaEventElapsedTime(ms, e->ev0, e->ev1), e->err);
  return PHX_OK;
}

phx_status phx_profile_enable(phx_engine* e, int32_t on) {
  if (!e) return PHX_E_ARG;
  e->profile = on != 0;
  e->prof_used = 0;
  return PHX_OK;
}

phx_status phx_profile_read(phx_engine* e, float* ms_by_class, int32_t* launches_by_class) {
  if (!e || !ms_by_class || !launches_by_class) return PHX_E_ARG;
  cudaSetDevice(e->device);
  PHX_CUDA_TRY(cudaStreamSynchronize(e->stream), e->err);
  for (int i = 0; i < KC_COUNT; ++i) { ms_by_class[i] = 0.f; launches_by_class[i] = 0; }
  float sub_ms[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int sub_n[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int res_seen = 0;
  for (size_t i = 0; i < e->prof_used; ++i) {
    float ms = 0.f;
    PHX_CUDA_TRY(cudaEventElapsedTime(&ms, e->prof_events[i].second.first, e->prof_events[i].second.second), e->err);
    const int cls = e->prof_events[i].first & 0xff;
    int sub = (e->prof_events[i].first >> 8) & 0xff;
    ms_by_class[cls] += ms;
    launches_by_class[cls] += 1;
    if (cls == KC_GEMM && sub > 0) {
      // the two residual GEMMs of a layer alternate: out-projection first, then the FFN down-projection
      if (sub - 1 == EPI_RESIDUAL) sub = (res_seen++ & 1) ? 6 : 5;
      sub_ms[sub & 7] += ms; sub_n[sub & 7] += 1;
    }
  }
  if (e->gemm_counters) {
    unsigned long long h[32];
    PHX_CUDA_TRY(cudaMemcpy(h, e->gemm_counters, sizeof(h), cudaMemcpyDeviceToHost), e->err);
    const char* role[4] = {"qkv", "out", "up", "down"};
    for (int r = 0; r < 4; ++r)
      fprintf(stderr, "[phx gemm counters] %s: MMA issuer waiting for operands %.1f%%, for a free accumulator %.1f%%\n", role[r],
              100.0 * h[8 * r + 1] / (double)(h[8 * r] ? h[8 * r] : 1), 100.0 * h[8 * r + 2] / (double)(h[8 * r] ? h[8 * r] : 1));
  }
#ifdef PHX_DIAGNOSTICS
  if (getenv("PHX_PROF_GEMM")) {   // diagnostics: GEMM time of the last forward by role
    fprintf(stderr, "[phx gemm breakdown] qkv(store) %.3f ms/%d  qkv(rope) %.3f ms/%d  up(gelu) %.3f ms/%d  out(res) %.3f ms/%d  down(res) %.3f ms/%d\n",
            sub_ms[1 + EPI_STORE], sub_n[1 + EPI_STORE], sub_ms[1 + EPI_ROPE], sub_n[1 + EPI_ROPE], sub_ms[1 + EPI_GELU],
            sub_n[1 + EPI_GELU], sub_ms[5], sub_n[5], sub_ms[6], sub_n[6]);
  }
#else
  (void)sub_ms; (void)sub_n;
#endif
  return PHX_OK;
}

phx_status phx_mark(phx_engine* e, int32_t slot) {
  if (!e || slot < 0 || slot > 7) return PHX_E_ARG;
  cudaSetDevice(e->device);
  if (!e->marks[slot]) PHX_CUDA_TRY(cudaEventCreate(&e->marks[slot]), e->err);
  PHX_CUDA_TRY(cudaEventRecord(e->marks[slot], e->stream), e->err);
  return PHX_OK;
}

phx_status phx_mark_wait(phx_engine* e, int32_t slot) {
  if (!e || slot < 0 || slot > 7) return PHX_E_ARG;
  if (!e->marks[slot]) return PHX_OK;   // never recorded: nothing to wait for
  PHX_CUDA_TRY(cudaEventSynchronize(e->marks[slot]), e->err);
  return PHX_OK;
}

phx_status phx_elapsed_ms(phx_engine* e, int32_t from_slot, int32_t to_slot, float* ms) {
  if (!e || !ms || from_slot < 0 || from_slot > 7 || to_slot < 0 || to_slot > 7 || !e->marks[from_slot] || !e->marks[to_slot]) return PHX_E_ARG;
  PHX_CUDA_TRY(cudaEventSynchronize(e->marks[to_slot]), e->err);
  PHX_CUDA_TRY(cudaEventElapsedTime(ms, e->marks[from_slot], e->marks[to_slot]), e->err);
  return PHX_OK;
}

phx_status phx_last_launch_count(phx_engine* e, int32_t* n) {
  if (!e || !n) return PHX_E_ARG;
  *n = e->last_launches;
  return PHX_OK;
}

phx_status phx_debug_read(phx_engine* e, const char* what, void* host, size_t nbytes) {
  if (!e || !what || !host) return PHX_E_ARG;
  cudaSetDevice(e->device);
  const std::string w(what);
  const size_t M = (size_t)e->last_batch * e->T;
  const void* src = nullptr; size_t avail = 0;
  if (w == "hidden" && e->fp32) { src = e->x32; avail = M * e->D * 4; }   // full-precision path: fp32 rows
  else if (w == "hidden") { src = e->x; avail = M * e->D * 2; }
  else if (w == "seg") { src = e->seg; avail = M * 4; }
  else if (w == "attn") { src = e->attn; avail = M * e->HD * 2; }
  else if (w == "qkv") { src = e->qkv; avail = M * e->QW * 2; }
  else if (w == "tokens" && e->debug_taps) { src = e->tokens; avail = M * e->D * 2; }
  else if (w == "hashes" && e->debug_taps) { src = e->hashes; avail = M * 2 * e->cfg.item.num_hashes * 4; }
  else { e->err = "phx_debug_read: unknown tap (tokens / hashes need PHX_DEBUG_TAPS=1): " + w; return PHX_E_ARG; }
  if (nbytes > avail) { e->err = "phx_debug_read: more bytes requested than the tap holds"; return PHX_E_ARG; }
  PHX_CUDA_TRY(cudaStreamSynchronize(e->stream), e->err);
  PHX_CUDA_TRY(cudaMemcpy(host, src, nbytes, cudaMemcpyDeviceToHost), e->err);
  return PHX_OK;
}

phx_status phx_hash_ids_device(phx_engine* e, int32_t family, const int64_t* ids_dev, int64_t n, int32_t* out_dev) {
  if (!e || family < 0 || family > 3 || n < 0) return PHX_E_ARG;
  cudaSetDevice(e->device);
  long long off[5];
  region_offsets(e->cfg, &off[0], &off[1], &off[2], &off[3], &off[4]);
  const phx_hash_family* fams[4] = {&e->cfg.user, &e->cfg.item, &e->cfg.author, &e->cfg.ip};
  return hash_ids_launch(to_dev(*fams[family], (int)off[family]), (const long long*)ids_dev, n, out_dev, e->stream, e->err);
}

phx_status phx_gather_sum_device(phx_engine* e, int32_t family, const int64_t* ids_dev, int64_t n, uint16_t* out_dev) {
  if (!e || family < 0 || family > 3 || n < 0) return PHX_E_ARG;
  cudaSetDevice(e->device);
  long long off[5];
  region_offsets(e->cfg, &off[0], &off[1], &off[2], &off[3], &off[4]);
  const phx_hash_family* fams[4] = {&e->cfg.user, &e->cfg.item, &e->cfg.author, &e->cfg.ip};
  PHX_CUDA_TRY(cudaEventRecord(e->ev0, e->stream), e->err);
  if (!shards_complete(e)) return PHX_E_STATE;
  phx_status s = gather_sum_launch(to_dev(*fams[family], (int)off[family]), table_view(e), e->D,
                                   (const long long*)ids_dev, n, (bf16*)out_dev, e->stream, e->err);
  if (s) return s;
  PHX_CUDA_TRY(cudaEventRecord(e->ev1, e->stream), e->err);
  return PHX_OK;
}

phx_status phx_user_tower_device(phx_engine* e, const phx_rank_batch* bd, float* users_dev) {
  if (!e || !bd || !users_dev) return PHX_E_ARG;
  if (bd->batch < 0 || bd->batch > e->cfg.max_batch) { e->err = "batch exceeds max_batch"; return PHX_E_CAPACITY; }
  if (!batch_arrays_present(e, bd, false, "phx_user_tower_device")) return PHX_E_ARG;
  if (!params_complete(e, false) || !shards_complete(e)) return PHX_E_STATE;
  cudaSetDevice(e->device);
  const int B = bd->batch;
  e->last_batch = B; e->last_launches = 0; e->prof_used = 0;
  if (B == 0) return PHX_OK;
  PHX_CUDA_TRY(cudaEventRecord(e->ev0, e->stream), e->err);
  phx_status s;
  if ((s = refresh_folded(e))) return s;
  // history only: tokens laid out [B, S]; every valid token is "history" so attention is full among them
  e->cur_pack = nullptr;
  if ((s = build_tokens(e, bd, B, 0))) return s;
  if ((s = run_trunk(e, B, e->S, e->S, e->S))) return s;
  { ProfScope ps(e, KC_HEADS); if ((s = tower_pool_launch(e->fp32 ? (const void*)e->x32 : (const void*)e->x, e->final_norm, e->seg, B, e->S, e->D, e->cfg.rms_eps, users_dev, e->stream, e->err, e->fp32))) return s; }
  e->last_launches++;
  PHX_CUDA_TRY(cudaEventRecord(e->ev1, e->stream), e->err);
  return PHX_OK;
}

phx_status phx_ranker_attention_device(int32_t device, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                       const int32_t* seg, uint16_t* out, int32_t B, int32_t T, int32_t Hq,
                                       int32_t Hkv, int32_t dh, int32_t hist_len, float sm_scale, float cap,
                                       int32_t cap_method, float* device_ms) {
  std::string err;
  if (cudaSetDevice(device) != cudaSuccess) { set_global_error("cudaSetDevice failed"); return PHX_E_CUDA; }
  AttnArgs aa;
  aa.q = (const bf16*)q; aa.k = (const bf16*)k; aa.v = (const bf16*)v;
  aa.q_tok_stride = (long long)Hq * dh; aa.k_tok_stride = aa.v_tok_stride = (long long)Hkv * dh;
  aa.q_head_stride = aa.k_head_stride = aa.v_head_stride = dh;
  aa.out = (bf16*)out; aa.seg = seg; aa.B = B; aa.T = T; aa.Hq = Hq; aa.Hkv = Hkv; aa.dh = dh; aa.hist_len = hist_len;
  aa.sm_scale = sm_scale; aa.cap = cap; aa.cap_method = cap > 0.f ? cap_method : 0;
  int* flag = nullptr;
  if (cudaMalloc(&flag, 2 * sizeof(int)) != cudaSuccess) { set_global_error("cudaMalloc failed"); return PHX_E_CUDA; }
  cudaMemset(flag, 0, 2 * sizeof(int));
  aa.err_flag = flag;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0, 0);
  phx_status s = ranker_attention_launch(aa, 0, err);
  cudaEventRecord(e1, 0);
  cudaError_t ce = cudaEventSynchronize(e1);
  if (s == PHX_OK && ce != cudaSuccess) { err = cudaGetErrorString(ce); s = PHX_E_CUDA; }
  if (s == PHX_OK && device_ms) cudaEventElapsedTime(device_ms, e0, e1);
  if (s == PHX_OK) {
    int hflag = 0;
    cudaMemcpy(&hflag, flag, sizeof(int), cudaMemcpyDeviceToHost);
    if (hflag) { err = "a bounded device-side wait ran out (attention pipeline)"; s = PHX_E_TIMEOUT; }
  }
  cudaFree(flag);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  if (s) set_global_error(err);
  return s;
}

phx_status phx_gemm_device(int32_t device, const uint16_t* A, const uint16_t* Wt, const uint16_t* R, uint16_t* C,
                           int64_t M, int32_t N, int32_t K, int32_t epilogue, int32_t impl, float* device_ms) {
  std::string err;
  if (cudaSetDevice(device) != cudaSuccess) { set_global_error("cudaSetDevice failed"); return PHX_E_CUDA; }
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, device);
  int* flag = nullptr;
  if (cudaMalloc(&flag, 2 * sizeof(int)) != cudaSuccess) { set_global_error("cudaMalloc failed"); return PHX_E_CUDA; }
  cudaMemset(flag, 0, 2 * sizeof(int));
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  phx_status s = PHX_OK;
  unsigned long long* ctr = nullptr;   // PHX_GEMM_COUNTERS=1: print where the MMA issuer waited (diagnostics)
  if (impl == 1) {
    cudaEventRecord(e0, 0);
    s = gemm_simt_launch((const bf16*)A, (const bf16*)Wt, (bf16*)C, (const bf16*)R, M, N, K, epilogue, 0, err);
    cudaEventRecord(e1, 0);
  } else {
    GemmPlan plan;
    s = gemm_plan_create(&plan, (const bf16*)A, (const bf16*)Wt, M, N, K, epilogue == 1 && K <= 1024, err, impl == 2 ? 0 : -1);
#ifdef PHX_DIAGNOSTICS
    if (getenv("PHX_GEMM_COUNTERS")) { cudaMalloc(&ctr, 64); cudaMemset(ctr, 0, 64); plan.counters = ctr; }
#endif
    cudaEventRecord(e0, 0);
    if (s == PHX_OK && (epilogue < 0 || epilogue > 2)) { err = "phx_gemm_device: epilogue must be 0, 1 or 2"; s = PHX_E_ARG; }
    if (s == PHX_OK) s = gemm_launch(plan, (const bf16*)A, (bf16*)C, (const bf16*)R, M, epilogue, nullptr, nullptr, flag, prop.multiProcessorCount, 0, err);
    cudaEventRecord(e1, 0);
  }
  cudaError_t ce = cudaEventSynchronize(e1);
  if (s == PHX_OK && ce != cudaSuccess) { err = cudaGetErrorString(ce); s = PHX_E_CUDA; }
  if (s == PHX_OK && device_ms) cudaEventElapsedTime(device_ms, e0, e1);
  int hflag = 0;
  if (s == PHX_OK) {
    cudaMemcpy(&hflag, flag, sizeof(int), cudaMemcpyDeviceToHost);
    if (hflag) { err = "a bounded device-side wait ran out (GEMM pipeline)"; s = PHX_E_TIMEOUT; }
  }
  if (ctr) {
    unsigned long long h[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    cudaMemcpy(h, ctr, 64, cudaMemcpyDeviceToHost);
    fprintf(stderr, "[phx gemm timeline, CTA 0] entry -> first MMA wait %.1f us, MMA window %.1f us, last MMA issued -> CTA done %.1f us\n",
            (h[4] - h[3]) * 1e-3, (h[5] - h[4]) * 1e-3, (h[6] - h[5]) * 1e-3);
    fprintf(stderr, "[phx gemm counters] MMA issuer cycles (sum over CTAs): total %llu, waiting for operands %llu (%.1f%%), "
            "waiting for a free accumulator %llu (%.1f%%)\n", h[0], h[1], 100.0 * h[1] / (double)(h[0] ? h[0] : 1), h[2],
            100.0 * h[2] / (double)(h[0] ? h[0] : 1));
    cudaFree(ctr);
  }
  cudaFree(flag);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  if (s) set_global_error(err);
  return s;
}

// ---- multi-hash gather-sum over the row-sharded table, exchange owned by the library -------------------------------------
namespace {
struct GatherWs {
  int W = 1, H = 0, width = 0;
  long long max_req = 0, shard_rows = 0, table_slots = 0, recv_cap = 0;
  int *rows = nullptr, *slot = nullptr, *urows = nullptr, *upos = nullptr, *pos = nullptr, *send_rows = nullptr;
  int *counts = nullptr, *cursor = nullptr, *nu = nullptr, *counts_all = nullptr, *recv_rows = nullptr;
  int* counts_host = nullptr;
  unsigned long long* table = nullptr;
  bf16 *gathered = nullptr, *landing = nullptr;
  bf16* peer_landing[PHX_MAX_SHARDS] = {nullptr};
  cudaEvent_t ev[9] = {};
};

// step 0: unmap the peers' landing buffers; step 1 (after every rank has done step 0): free this rank's memory
void gather_ws_free(void* p, int step) {
  GatherWs* w = static_cast<GatherWs*>(p);
  if (step == 0) {
    for (int r = 0; r < w->W; ++r)
      if (w->peer_landing[r] && w->peer_landing[r] != w->landing) { cudaIpcCloseMemHandle(w->peer_landing[r]); w->peer_landing[r] = nullptr; }
    return;
  }
  for (void* q : {(void*)w->rows, (void*)w->slot, (void*)w->urows, (void*)w->upos, (void*)w->pos, (void*)w->send_rows, (void*)w->counts,
                  (void*)w->cursor, (void*)w->nu, (void*)w->counts_all, (void*)w->recv_rows, (void*)w->table, (void*)w->gathered,
                  (void*)w->landing})
    if (q) cudaFree(q);
  if (w->counts_host) cudaFreeHost(w->counts_host);
  for (auto e : w->ev) if (e) cudaEventDestroy(e);
  delete w;
}
}  // namespace

phx_status phx_gather_sharded_setup(phx_comm* cm, phx_engine* e, int64_t max_ids, double recv_factor) {
  if (!cm || !e || max_ids <= 0 || recv_factor < 1.0) { set_global_error("phx_gather_sharded_setup: bad argument"); return PHX_E_ARG; }
  if (e->table_world != cm->world || e->table_rank != cm->rank || e->device != cm->device) {
    cm->err = "phx_gather_sharded_setup: the engine's table_world / table_rank / device do not match the communicator";
    return PHX_E_ARG;
  }
  cudaSetDevice(e->device);
  if (cm->gather_ws) {      // a second set-up: every rank unmaps, then every rank frees
    cm->gather_ws_free(cm->gather_ws, 0);
    phx_status bs = phx_comm_barrier(cm, nullptr);
    if (bs) return bs;
    cm->gather_ws_free(cm->gather_ws, 1);
    cm->gather_ws = nullptr;
  }
  GatherWs* w = new GatherWs();
  cm->gather_ws = w; cm->gather_ws_free = gather_ws_free;
  const int W = cm->world, H = e->cfg.item.num_hashes;
  w->W = W; w->H = H; w->width = e->D; w->shard_rows = e->shard_rows;
  w->max_req = (long long)max_ids * H;
  w->table_slots = 2; while (w->table_slots < 2 * w->max_req) w->table_slots *= 2;
  w->recv_cap = (long long)(recv_factor * (double)w->max_req) + 1;
  const size_t nr = (size_t)w->max_req;
#define GA(ptr, bytes) PHX_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&(ptr)), (bytes)), cm->err)
  GA(w->rows, nr * 4); GA(w->slot, nr * 4); GA(w->urows, nr * 4); GA(w->upos, nr * 4); GA(w->pos, nr * 4); GA(w->send_rows, nr * 4);
  GA(w->counts, 64 * 4); GA(w->cursor, 64 * 4); GA(w->nu, 4); GA(w->counts_all, ((size_t)W * W + 4) * 4);
  GA(w->recv_rows, (size_t)w->recv_cap * 4); GA(w->table, (size_t)w->table_slots * 8);
  GA(w->gathered, (size_t)w->recv_cap * w->width * 2); GA(w->landing, nr * w->width * 2);
#undef GA
  PHX_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&w->counts_host), ((size_t)W * W + 4) * 4), cm->err);
  for (auto& ev : w->ev) PHX_CUDA_TRY(cudaEventCreate(&ev), cm->err);
  // every rank maps every other rank's landing buffer: handles travel through one all-gather
  w->peer_landing[cm->rank] = w->landing;
  if (W > 1) {
    cudaIpcMemHandle_t mine;
    PHX_CUDA_TRY(cudaIpcGetMemHandle(&mine, w->landing), cm->err);
    uint8_t* hbuf = nullptr;
    PHX_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&hbuf), (size_t)(W + 1) * sizeof(mine)), cm->err);
    PHX_CUDA_TRY(cudaMemcpy(hbuf + (size_t)W * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice), cm->err);
    phx_status s = comm_check(cm, cm->api->AllGather(hbuf + (size_t)W * sizeof(mine), hbuf, sizeof(mine), ncclUint8, cm->comm, 0), "ncclAllGather (handles)");
    if (s) { cudaFree(hbuf); return s; }
    std::vector<cudaIpcMemHandle_t> all(W);
    cudaError_t ce = cudaMemcpy(all.data(), hbuf, (size_t)W * sizeof(mine), cudaMemcpyDeviceToHost);   // waits for the collective
    cudaFree(hbuf);
    if (ce != cudaSuccess) { cm->err = std::string("handle exchange: ") + cudaGetErrorString(ce); return PHX_E_CUDA; }
    for (int r = 0; r < W; ++r) {
      if (r == cm->rank) continue;
      void* p = nullptr;
      PHX_CUDA_TRY(cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess), cm->err);
      w->peer_landing[r] = static_cast<bf16*>(p);
    }
  }
  return phx_comm_barrier(cm, nullptr);
}

phx_status phx_gather_sum_sharded(phx_comm* cm, phx_engine* e, int32_t family, const int64_t* ids_dev, int64_t n, uint16_t* out_dev,
                                  void* stream) {
  return phx_gather_sum_sharded_multi(cm, e, 1, &family, &n, ids_dev, out_dev, stream);
}

phx_status phx_gather_sum_sharded_multi(phx_comm* cm, phx_engine* e, int32_t nseg, const int32_t* seg_family, const int64_t* seg_count,
                                        const int64_t* ids_dev, uint16_t* out_dev, void* stream) {
  if (!cm || !e || nseg < 1 || nseg > 16 || !seg_family || !seg_count) { set_global_error("phx_gather_sum_sharded: bad argument"); return PHX_E_ARG; }
  int64_t n = 0;
  const phx_hash_family* fams[4] = {&e->cfg.user, &e->cfg.item, &e->cfg.author, &e->cfg.ip};
  for (int i = 0; i < nseg; ++i) {
    if (seg_family[i] < 0 || seg_family[i] > 3 || seg_count[i] < 0) { set_global_error("phx_gather_sum_sharded: bad family or count"); return PHX_E_ARG; }
    if (seg_count[i] > 0 && fams[seg_family[i]]->num_hashes != e->cfg.item.num_hashes) {
      set_global_error("phx_gather_sum_sharded: every family of a call must have the engine's item hash count"); return PHX_E_ARG;
    }
    n += seg_count[i];
  }
  if (n > 0 && (!ids_dev || !out_dev)) { set_global_error("phx_gather_sum_sharded: bad argument"); return PHX_E_ARG; }
  GatherWs* w = static_cast<GatherWs*>(cm->gather_ws);
  if (!w) { cm->err = "phx_gather_sum_sharded: call phx_gather_sharded_setup first"; return PHX_E_STATE; }
  const int W = w->W, H = w->H, rank = cm->rank;
  const long long nreq = n * H;
  if (nreq > w->max_req) { cm->err = "phx_gather_sum_sharded: more ids than the set-up allowed for"; return PHX_E_CAPACITY; }
  cudaSetDevice(e->device);
  cudaStream_t st = (cudaStream_t)stream;
  long long off[5];
  region_offsets(e->cfg, &off[0], &off[1], &off[2], &off[3], &off[4]);
  phx_status s;
  auto mark = [&](int i) { cudaEventRecord(w->ev[i], st); };
  mark(0);
  // requester: ids -> rows (run by run, each with its family's constants and region) -> distinct rows -> grouped by
  // owner; nothing here waits on the host
  {
    int64_t at = 0;
    for (int i = 0; i < nseg; ++i) {
      const int f = seg_family[i];
      if (seg_count[i] > 0 &&
          (s = hash_ids_launch(to_dev(*fams[f], (int)off[f]), (const long long*)ids_dev + at, seg_count[i], w->rows + at * H, st, cm->err))) return s;
      at += seg_count[i];
    }
  }
  if ((s = phx_shard_dedup(w->rows, nreq, (uint64_t*)w->table, w->table_slots, w->slot, w->urows, w->nu, st))) { cm->err = phx_global_error(); return s; }
  if ((s = shard_bucket_launch(w->urows, nreq, w->nu, w->shard_rows, W, w->counts, w->cursor, w->send_rows, w->upos, st))) { cm->err = phx_global_error(); return s; }
  if ((s = phx_shard_dedup_expand(w->slot, (const uint64_t*)w->table, w->upos, nreq, w->pos, st))) { cm->err = phx_global_error(); return s; }
  mark(1);
  // every rank learns every rank's per-owner counts: one all-gather, one copy to the host, the only host wait
  if ((s = comm_check(cm, cm->api->AllGather(w->counts, w->counts_all, W, ncclInt32, cm->comm, st), "ncclAllGather (counts)"))) return s;
  PHX_CUDA_TRY(cudaMemcpyAsync(w->counts_host, w->counts_all, (size_t)W * W * 4, cudaMemcpyDeviceToHost, st), cm->err);
  PHX_CUDA_TRY(cudaStreamSynchronize(st), cm->err);
  mark(2);
  const int* all = w->counts_host;                 // all[requester * W + owner]
  long long send_off[PHX_MAX_SHARDS + 1], recv_off[PHX_MAX_SHARDS + 1], their_off[PHX_MAX_SHARDS];
  send_off[0] = recv_off[0] = 0;
  for (int p = 0; p < W; ++p) {
    send_off[p + 1] = send_off[p] + all[rank * W + p];
    recv_off[p + 1] = recv_off[p] + all[p * W + rank];
    long long o = 0;
    for (int q = 0; q < rank; ++q) o += all[p * W + q];
    their_off[p] = o;                              // where requester p keeps the bucket of rows it asked of this rank
  }
  if (recv_off[W] > w->recv_cap) {
    cm->err = "phx_gather_sum_sharded: this rank was asked for " + std::to_string(recv_off[W]) + " rows, the set-up allows " +
              std::to_string(w->recv_cap) + " (raise recv_factor)";
    return PHX_E_CAPACITY;
  }
  // row numbers to their owners
  if ((s = comm_check(cm, cm->api->GroupStart(), "ncclGroupStart"))) return s;
  for (int i = 1; i < W; ++i) {
    const int to = (rank + i) % W, from = (rank - i + W) % W;
    if (all[rank * W + to] > 0 && (s = comm_check(cm, cm->api->Send(w->send_rows + send_off[to], (size_t)all[rank * W + to], ncclInt32, to, cm->comm, st), "ncclSend (row numbers)"))) return s;
    if (all[from * W + rank] > 0 && (s = comm_check(cm, cm->api->Recv(w->recv_rows + recv_off[from], (size_t)all[from * W + rank], ncclInt32, from, cm->comm, st), "ncclRecv (row numbers)"))) return s;
  }
  if ((s = comm_check(cm, cm->api->GroupEnd(), "ncclGroupEnd"))) return s;
  if (all[rank * W + rank] > 0)
    PHX_CUDA_TRY(cudaMemcpyAsync(w->recv_rows + recv_off[rank], w->send_rows + send_off[rank], (size_t)all[rank * W + rank] * 4, cudaMemcpyDeviceToDevice, st), cm->err);
  mark(3);
  // owner: per requester, gather its rows into a send block; the copy engines carry each finished block into the
  // requester's landing buffer (one copy per peer) while the next block is gathered
  const size_t row_bytes = (size_t)w->width * 2;
  int used = 0;
  for (int i = 1; i < W; ++i) {
    const int p = (rank + i) % W;
    const long long cnt = all[p * W + rank];
    if (cnt == 0) continue;
    bf16* block = w->gathered + recv_off[p] * w->width;
    if ((s = phx_shard_gather_rows((const uint16_t*)e->table, w->shard_rows, w->recv_rows + recv_off[p], cnt, w->width, (uint16_t*)block, st))) { cm->err = phx_global_error(); return s; }
    PHX_CUDA_TRY(cudaEventRecord(cm->ev_fork, st), cm->err);
    cudaStream_t cs = cm->side[used % 4];
    PHX_CUDA_TRY(cudaStreamWaitEvent(cs, cm->ev_fork, 0), cm->err);
    PHX_CUDA_TRY(cudaMemcpyAsync(w->peer_landing[p] + their_off[p] * w->width, block, (size_t)cnt * row_bytes, cudaMemcpyDefault, cs), cm->err);
    ++used;
  }
  if (all[rank * W + rank] > 0 &&
      (s = phx_shard_gather_rows((const uint16_t*)e->table, w->shard_rows, w->recv_rows + recv_off[rank], all[rank * W + rank], w->width,
                                 (uint16_t*)(w->landing + their_off[rank] * w->width), st))) { cm->err = phx_global_error(); return s; }
  mark(4);
  for (int i = 0; i < (used < 4 ? used : 4); ++i) {
    PHX_CUDA_TRY(cudaEventRecord(cm->ev_join[i], cm->side[i]), cm->err);
    PHX_CUDA_TRY(cudaStreamWaitEvent(st, cm->ev_join[i], 0), cm->err);
  }
  mark(5);
  // every rank's copies have landed before any rank sums
  if (W > 1 && (s = comm_check(cm, cm->api->AllReduce(cm->fence, cm->fence, 1, ncclInt32, ncclSum, cm->comm, st), "ncclAllReduce (fence)"))) return s;
  mark(6);
  if ((s = phx_shard_sum_rows((const uint16_t*)w->landing, w->pos, n, H, w->width, out_dev, st))) { cm->err = phx_global_error(); return s; }
  mark(7);
  return PHX_OK;
}

// Device time of the phases of the last phx_gather_sum_sharded call on this rank (waits for it): hash + dedup + bucket,
// counts exchange (with the host wait), row numbers, owner-side gathers, the rest of the copies, fence, sum.  Seven floats.
phx_status phx_gather_sharded_phase_ms(phx_comm* cm, float* ms7) {
  if (!cm || !ms7 || !cm->gather_ws) return PHX_E_ARG;
  GatherWs* w = static_cast<GatherWs*>(cm->gather_ws);
  PHX_CUDA_TRY(cudaEventSynchronize(w->ev[7]), cm->err);
  for (int i = 0; i < 7; ++i) PHX_CUDA_TRY(cudaEventElapsedTime(&ms7[i], w->ev[i], w->ev[i + 1]), cm->err);
  return PHX_OK;
}

}  // extern "C"
