// Shared declarations of the Phoenix B200 engine (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>

#include "../../include/phoenix_b200.h"

namespace phx {

typedef __nv_bfloat16 bf16;

// ---- error plumbing ---------------------------------------------------------------------------
void set_global_error(const std::string& msg);

#define PHX_CUDA_TRY(call, errstr)                                                               \
  do {                                                                                           \
    cudaError_t _e = (call);                                                                     \
    if (_e != cudaSuccess) {                                                                     \
      (errstr) = std::string(#call) + ": " + cudaGetErrorString(_e) + " (" + __FILE__ + ":" +    \
                 std::to_string(__LINE__) + ")";                                                 \
      return PHX_E_CUDA;                                                                         \
    }                                                                                            \
  } while (0)

// ---- which kernel variant a launch took (host-side counters, read through phx_dispatch_counts) -------------------
enum DispatchKind {
  DK_ATTN_STRIP = 0,     // resident-history mma.sync kernel (head dim 64, <= 128 history keys)
  DK_ATTN_STREAM = 1,    // streaming mma.sync kernel
  DK_ATTN_TC = 2,        // tcgen05 / TMEM streaming kernel
  DK_ATTN_RESIDENT = 3,  // tcgen05 / TMEM resident-history kernel
  DK_GEMM_PAIR256 = 4,   // tcgen05 GEMM, CTA pairs, 256-column tiles
  DK_GEMM_PAIR128 = 5,
  DK_GEMM_CTA256 = 6,    // tcgen05 GEMM, one CTA per tile
  DK_GEMM_CTA128 = 7,
  DK_GEMM_SIMT = 8,
  DK_SCAN_TC = 9,        // tcgen05 corpus scan
  DK_SCAN_MMA = 10,      // mma.sync corpus scan
  DK_TOPK_EXACT = 11,    // exact-threshold passes of the top-k (the sampled pivot missed)
  DK_ATTN_PINGPONG = 12, // tcgen05 / TMEM resident-history kernel with two softmax warpgroups
  DK_COUNT = 13
};
void dispatch_note(int kind);

// ---- bf16 <-> f32 on device -------------------------------------------------------------------
__device__ __forceinline__ float bf2f(bf16 x) { return __bfloat162float(x); }
__device__ __forceinline__ bf16 f2bf(float x) { return __float2bfloat16_rn(x); }
__device__ __forceinline__ float round_bf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

// GELU, tanh form.  tanh.approx (one MUFU op, abs error ~5e-4) is far below the bf16 rounding applied to the
// result, and keeps the GEMM epilogue off the critical path.
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float c = 0.7978845608028654f;  // sqrt(2/pi)
  float inner = c * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(inner));
  return 0.5f * x * (1.0f + t);
}

// ---- GEMM ---------------------------------------------------------------------------------------
enum GemmEpilogue { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_GELU = 2, EPI_ROPE = 3 };

// RoPE fused into the epilogue of the merged QKV projection: applied to the q and k head parts
// (column part p of width dh is q or k when p % group <= g; group = g + 2, g = q heads per kv head).
struct GemmRope {
  const float* cos_tab;  // [pos_cap + 1, dh / 2]
  const float* sin_tab;
  int T;                 // tokens per request: position = min(row % T, pos_cap)
  int pos_cap;
  int dh;                // 32 or 64
  int group, g;
  // split token layout (all history rows, then all candidate rows): GEMM row r is token row r + row_offset; rows
  // below split_rows are history rows of `T` per request, the rows from split_rows on sit at position pos_cap.
  // split_rows = 0: plain layout.
  long long row_offset = 0, split_rows = 0;
  const int* pos_rows = nullptr;   // packed rows: position of every token row (overrides the rule above)
};

// Token rows of a [B, S + C] batch.  Plain layout: row = b * T + t.  Split layout (engines with candidate-only tail
// layers): the B * S history rows first, then the B * C candidate rows, so that the GEMMs of a tail layer run over
// one contiguous block of candidate rows and leave the history block untouched.
__host__ __device__ inline long long token_row(int split, int B, int S, int T, int b, int t) {
  if (!split) return (long long)b * T + t;
  return t < S ? (long long)b * S + t : (long long)B * S + (long long)b * (T - S) + (t - S);
}

// Packed token rows (ragged batches): request b keeps only its first hist_cnt history slots and its first cand_cnt
// candidate slots (front-filled requests), the history rows of all requests back to back, then all candidate rows:
// row of history slot t = hist_off[b] + t, of candidate slot c = cand_base + cand_off[b] + c.  hist_off / cand_off are
// exclusive prefix sums with B + 1 entries.  off = null: not packed.
struct PackMap {
  const int* hist_off = nullptr;
  const int* cand_off = nullptr;
  long long cand_base = 0;
  __device__ __forceinline__ bool on() const { return hist_off != nullptr; }
  __device__ __forceinline__ int hist_cnt(int b) const { return hist_off[b + 1] - hist_off[b]; }
  __device__ __forceinline__ int cand_cnt(int b) const { return cand_off[b + 1] - cand_off[b]; }
  // row of position t of request b in its own packed coordinates (history 0..hist_cnt-1, then candidates)
  __device__ __forceinline__ long long row(int b, int t) const {
    const int hc = hist_cnt(b);
    return t < hc ? (long long)hist_off[b] + t : cand_base + cand_off[b] + (t - hc);
  }
};

// RMSNorm folded around a GEMM.  Consumer side (ss_in): the A rows are the raw residual stream, the norm's gain is
// folded into the weights, and the epilogue scales row r by rsqrt(sum_t ss_in[r][t] / D + eps) before rounding
// (x rstd g) W = rstd (x (g W)).  Producer side (ss_out, residual epilogue): the sum of squares of each new bf16
// residual row is left in ss_out[r][column slab] for the next consumer - one slot per 64-column slab, no atomics,
// so the statistics are deterministic.
struct GemmNorm {
  const float* ss_in;
  float* ss_out;
  int slots_in;
  float inv_d, eps;
};

// One GEMM problem bound to fixed buffers: C[M,N] = epi(A[M,K] @ Wt[N,K]^T).  The tensor maps
// are encoded once for (pointer, rows_max) and reused for every M <= rows_max.
struct GemmPlan {
  CUtensorMap map_a;
  CUtensorMap map_b;
  CUtensorMap map_b_narrow;   // W map for 128-column tiles, used when a call has too few wide tiles to fill the device
  bool has_narrow = false;
  CUtensorMap map_c;   // output map, re-encoded when the output pointer or M changes
  CUtensorMap map_r;   // residual map, likewise
  const bf16* c_ptr = nullptr; const bf16* r_ptr = nullptr;
  int64_t c_rows = -1, r_rows = -1;
  const bf16* A = nullptr;
  const bf16* Wt = nullptr;
  int64_t rows_max = 0;
  int64_t a_rows = 0;   // rows the A map was encoded over (rows_max, or the M of the call that moved A)
  int N = 0, K = 0, BN = 0;
  bool pair = false;   // two CTAs of a cluster share each 256-row tile (tcgen05 cta_group::2)
  bool ready = false;
  unsigned long long* counters = nullptr;  // optional device counters [8]: MMA issuer cycles total / waiting for
                                           // operands / waiting for a free accumulator (diagnostics)
};

// narrow_tiles: use 128 x 128 tiles even when N is a multiple of 256 (more output slab buffers; meant for
// residual GEMMs with a short K, which are bound by HBM rather than by the tensor pipe)
phx_status gemm_plan_create(GemmPlan* plan, const bf16* A, const bf16* Wt, int64_t rows_max, int N, int K,
                            bool narrow_tiles, std::string& err, int pair = -1);
// pair: 1 = CTA pairs share 256-row tiles (cta_group::2), 0 = one CTA per 128-row tile, -1 = pairs unless the
// environment says PHX_GEMM=cta1
// Launch on `stream`.  `R` is the residual (EPI_RESIDUAL) or null.  `err_flag` is a device int the
// kernel sets to 1 when a bounded wait ran out.
phx_status gemm_launch(GemmPlan& plan, const bf16* A, bf16* C, const bf16* R, int64_t M, int epilogue,
                       const GemmRope* rope, const GemmNorm* norm, int* err_flag, int num_sms, cudaStream_t stream,
                       std::string& err);
// Plain SIMT GEMM with the same epilogues (debug / cross-check path, selected by PHX_GEMM=simt).
phx_status gemm_simt_launch(const bf16* A, const bf16* Wt, bf16* C, const bf16* R, int64_t M, int N, int K,
                            int epilogue, cudaStream_t stream, std::string& err);

// ---- embedding ----------------------------------------------------------------------------------
struct HashFamilyDev {
  long long scales[PHX_MAX_HASHES];
  long long biases[PHX_MAX_HASHES];
  long long modulus;
  long long buckets_m1;  // table_size - 1
  unsigned long long magic_mod;  // floor((2^64 - 1) / modulus): division-free remainder
  unsigned long long magic_bkt;  // floor((2^64 - 1) / buckets_m1)
  int offset;            // region offset in the unified table
  int num_hashes;
};

// The unified embedding table, possibly row-sharded over `world` devices in contiguous ranges: global row r lives
// on shard r / rows_per_shard at local row r % rows_per_shard (the reference's row_emb ownership rule,
// phoenix/xrex/cuda/row_emb/src/row_emb_kernel.hpp:19-25).  base[s] is a pointer this device can load from:
// its own shard, or a peer's shard mapped over NVLink.  world == 1: one shard holding every row.
#define PHX_MAX_SHARDS 16
struct TableView {
  const bf16* base[PHX_MAX_SHARDS];
  long long total_rows;
  unsigned int rows_per_shard;
  int world;
  __device__ __forceinline__ const bf16* row_ptr(long long row, int D) const {
    if (row < 0 || row >= total_rows) row = 0;  // out of range -> row 0 (emb_table.rs:134-137)
    if (world == 1) return base[0] + row * D;
    const unsigned int r = (unsigned int)row;
    const unsigned int s = r / rows_per_shard;
    return base[s] + (long long)(r - s * rows_per_shard) * D;
  }
};

struct TokenBuildArgs {
  const long long* hist_post;
  const long long* hist_author;
  const int* hist_actions;
  const int* hist_surfaces;
  const long long* cand_post;
  const long long* cand_author;
  TableView table;
  const bf16* action_table;
  const bf16* surface_table;
  int num_action_types, num_surfaces;
  HashFamilyDev item, author;
  int B, S, C, D;
  float input_scale;
  bf16* x;         // [B,T,D] scaled tokens
  float* row_ss;   // optional [B*T, ss_slots]: sum of squares of each x row in slot 0, zeros in the others
  int ss_slots;
  bf16* tokens;    // optional [B,T,D] unscaled gather-sum output
  int* hashes;     // optional [B,T,2H]
  int* seg;        // [B,T] 1 / -1 / 0
  // row-sharded table, exchange done outside the kernel: rows_only = just write the [B,T,2H] unified-table rows to
  // `hashes` and stop; landing / pos = take slot j of a token from landing[pos[tok*2H + j]] instead of the table
  int rows_only = 0;
  int split = 0;   // x / seg / row_ss rows in split layout (token_row)
  // pre-hashed input (the batch-prep buffers of the reference as they are): unified-table rows [B,S,H] / [B,C,H] per
  // feature, 0 = padding; when pre_hist_post is set the ids are not read and nothing is hashed
  const int* pre_hist_post = nullptr; const int* pre_hist_author = nullptr;
  const int* pre_cand_post = nullptr; const int* pre_cand_author = nullptr;
  // projected tokens: when concat_hist is set the kernel only lays the gathered rows side by side -
  // concat_hist [B*S, (2H+2)*D], concat_cand [B*C, 2H*D] - and writes the segment ids
  bf16* concat_hist = nullptr; bf16* concat_cand = nullptr;
  int action_multi_hot = 0;   // hist_actions are bit sets and action_table is one [D] vector cut into num_action_types chunks
  PackMap pack;           // packed rows: slots past a request's counts are skipped altogether
  float* x32 = nullptr;   // full-precision path: bf16(sum) * input_scale kept in fp32 here (x is then not written)
  const bf16* landing = nullptr;
  const int* pos = nullptr;
  // ---- batch-prep buffers beyond posts and authors (pre-hashed input only) ----
  // P user-prefix tokens (0 or 1) in front of every request's history: S counts them, the history input arrays hold
  // S - P slots.  User token = rows user_hashes [B,Hu] (side by side in concat_user [B, Hu*D], or summed) plus the sum of
  // the rows user_ip_hashes [B,Hip] (NULL: none); valid when user_hashes[b,0] != 0.
  int P = 0, Hu = 0, Hip = 0;
  const int* user_hashes = nullptr; const int* user_ip_hashes = nullptr;
  bf16* concat_user = nullptr;
  const unsigned char* hist_actions_bool = nullptr;   // bool [B,S-P,num_action_types] in place of hist_actions
  const int* cand_surfaces = nullptr;                 // [B,C]: one more candidate slot, a row of surface_table
  // continuous history actions: token += bf16(gelu(norm(v) * w1) @ w2) per configured column of hist_cont [B,S-P,8]
  const float* hist_cont = nullptr;
  int n_cont = 0, cont_hidden = 0;
  int cont_index[PHX_MAX_HIST_CONT] = {0, 0, 0, 0};
  int cont_log[PHX_MAX_HIST_CONT] = {0, 0, 0, 0};
  float cont_scale[PHX_MAX_HIST_CONT] = {1.f, 1.f, 1.f, 1.f};
  const bf16* cont_w1[PHX_MAX_HIST_CONT] = {nullptr, nullptr, nullptr, nullptr};   // [hidden]
  const bf16* cont_w2[PHX_MAX_HIST_CONT] = {nullptr, nullptr, nullptr, nullptr};   // [hidden, D]
};
phx_status pack_plan_launch(const PackMap& pk, int B, int S, int C, int* pos_rows, int* out_index, cudaStream_t stream,
                            std::string& err);
phx_status finish_tokens_launch(const bf16* tok_user, const bf16* tok_hist, const bf16* tok_cand, const TokenBuildArgs& a,
                                cudaStream_t stream, std::string& err);
phx_status build_tokens_launch(const TokenBuildArgs& a, cudaStream_t stream, std::string& err);
phx_status hash_ids_launch(const HashFamilyDev& fam, const long long* ids, long long n, int* out, cudaStream_t stream,
                           std::string& err);
phx_status gather_sum_launch(const HashFamilyDev& fam, const TableView& table, int D,
                             const long long* ids, long long n, bf16* out, cudaStream_t stream, std::string& err);
phx_status table_fill_launch(bf16* table, long long row0, long long rows, int width, uint32_t seed, float amp,
                             cudaStream_t stream, std::string& err);
phx_status corpus_fill_launch(bf16* rows_ptr, long long global_row0, long long rows, int dim, uint32_t seed,
                              cudaStream_t stream, std::string& err);

// grouping of row requests by owning rank (shard_exchange.cu); n_dev: optional device-side request count (<= n_req)
phx_status shard_bucket_launch(const int* rows_dev, long long n_req, const int* n_dev, long long rows_per_shard, int world,
                               int* counts_dev, int* cursor_dev, int* send_rows_dev, int* pos_dev, cudaStream_t stream);

// ---- elementwise --------------------------------------------------------------------------------
// y = bf16(norm(x) * gain); with `res` non-null y = bf16(res + bf16(norm(x) * gain)).  y may alias x or res.
phx_status rmsnorm_launch(const bf16* x, const float* gain, bf16* y, const bf16* res, long long rows, int D, float eps,
                          cudaStream_t stream, std::string& err);
phx_status fold_gain_launch(const bf16* w_t, const float* gain, bf16* out, int N, int K, cudaStream_t stream,
                            std::string& err);
struct QkNormRopeArgs {
  bf16* qkv;             // [M, qkv_width], merged layout per kv group [q_0..q_{g-1}, k, v]
  long long M;
  int T, Hq, Hkv, dh;
  int pos_cap;           // position = min(t, pos_cap)
  int rotary, qk_norm;
  const float* q_gain;   // [Hq*dh] or null
  const float* k_gain;   // [Hkv*dh] or null
  const float* cos_tab;  // [pos_cap+1, dh/2]
  const float* sin_tab;
  long long row_offset = 0, split_rows = 0;   // split token layout, as in GemmRope
  const int* pos_rows = nullptr;              // packed rows, as in GemmRope
};
phx_status qknorm_rope_launch(const QkNormRopeArgs& a, cudaStream_t stream, std::string& err);

// ---- attention ----------------------------------------------------------------------------------
struct AttnArgs {
  const bf16* q; const bf16* k; const bf16* v;  // element strides below
  long long q_tok_stride, k_tok_stride, v_tok_stride;  // between consecutive tokens
  int q_head_stride, k_head_stride, v_head_stride;     // between consecutive heads
  // grouped-query layouts where the q heads of one kv group sit together (merged QKV: [q_0..q_{g-1}, k, v] per kv
  // head): q head h starts at (h / q_group) * q_group_stride + (h % q_group) * q_head_stride.  q_group = 1: h * q_head_stride
  int q_group = 1, q_group_stride = 0;
  __host__ __device__ long long q_col(int h) const {
    return q_group <= 1 ? (long long)h * q_head_stride : (long long)(h / q_group) * q_group_stride + (long long)(h % q_group) * q_head_stride;
  }
  bf16* out;             // [B,T,Hq,dh] dense
  const int* seg;        // [B,T]
  int B, T, Hq, Hkv, dh, hist_len;
  float sm_scale, cap;
  int cap_method;
  int* err_flag;         // device int raised by a bounded wait that ran out (tcgen05 path); null = mma.sync path only
  // Split token layout (token_row): q / k / v / out / seg rows are the B * hist_len history rows followed by the
  // candidate rows; mma.sync kernels only.  q_start > 0: query rows below it are not computed (candidate-only layers).
  int split = 0, q_start = 0;
  // Packed rows (PackMap): per-request history / candidate counts; T and hist_len are then the largest a request can
  // have (grid sizing), q_start > 0 means "history queries are not wanted".  mma.sync kernels only.
  PackMap pack;
};
// tcgen05 / TMEM kernel for head dims 64 and 128 (attention_sm100.cu); the mma.sync kernel covers the rest
bool ranker_attention_tc_supported(const AttnArgs& a);
phx_status ranker_attention_tc_launch(const AttnArgs& a, int* err_flag, cudaStream_t stream, std::string& err);
bool ranker_attention_pingpong_supported(const AttnArgs& a);
phx_status ranker_attention_pingpong_launch(const AttnArgs& a, int* err_flag, cudaStream_t stream, std::string& err);
phx_status ranker_attention_launch(const AttnArgs& a, cudaStream_t stream, std::string& err);
// One thread waits on an mbarrier that nothing ever signals, with the flag block's wait limit: the wait gives up, raises
// the flag and the kernel returns (the bounded-wait path of every tcgen05 kernel here, exercised on its own).
phx_status wait_selftest_launch(int* err_flag, cudaStream_t stream, std::string& err);

// ---- heads + blend ------------------------------------------------------------------------------
struct HeadsArgs {
  const bf16* x;          // trunk output [B,T,D]
  const float* final_gain;
  const bf16* unembed_t;  // [V+NC, D] (transposed, K-major)
  int B, T, S, C, D, V, NC;
  float eps, output_scale, final_logit_cap, dwell_norm_scale;
  phx_blend_spec blend;
  int has_blend;
  float* log_probs; float* continuous; double* scores;
  // packed rows: x holds `rows` candidate rows back to back and row r's outputs go to candidate slot out_index[r] of
  // the [B, C] output arrays (the other slots are left as they are)
  const int* out_index = nullptr;
  long long rows = 0;
};
phx_status heads_launch(const HeadsArgs& a, cudaStream_t stream, std::string& err);
// masked mean pool + L2 normalise of final-normed history rows -> f32 [B,D]; x bf16, or fp32 (nothing rounded) when
// x_is_f32
phx_status tower_pool_launch(const void* x, const float* final_gain, const int* seg, int B, int T, int D, float eps,
                             float* users, cudaStream_t stream, std::string& err, bool x_is_f32 = false);

// ---- full-precision path (fp32_path.cu): fp32 activations, SIMT kernels, plain [B, T] token rows -------------------
phx_status f32_rmsnorm_launch(const float* x, const float* gain, float* y, const float* res, long long rows, int D, float eps,
                              cudaStream_t stream, std::string& err);
phx_status f32_gemm_launch(const float* A, const bf16* Wt, float* C, const float* R, int64_t M, int N, int K, int epilogue,
                           cudaStream_t stream, std::string& err);
phx_status f32_qknorm_rope_launch(float* qkv, long long M, int T, int Hq, int Hkv, int dh, int pos_cap, int rotary, int qk_norm,
                                  const float* q_gain, const float* k_gain, const float* cos_tab, const float* sin_tab,
                                  cudaStream_t stream, std::string& err);
phx_status f32_attention_launch(const float* qkv, const int* seg, float* out, int B, int T, int Hq, int Hkv, int dh,
                                int hist_len, float sm_scale, float cap, int cap_method, cudaStream_t stream, std::string& err);
phx_status f32_heads_launch(const float* x, const HeadsArgs& a, cudaStream_t stream, std::string& err);

}  // namespace phx
