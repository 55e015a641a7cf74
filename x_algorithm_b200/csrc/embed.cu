// Multi-hash id -> unified-table row (phoenix/xrex/models/recsys_embedding.py:154-172, 282-331),
// row gather (xai-recsys-engine/src/emb_table.rs:124-140) and the fixed-order fp32 combine of the
// gathered rows into one token.  HBM-bound: one warp per token, 16-byte loads per lane, rows of one
// token read back to back and summed in slot order so the result does not depend on the launch shape.
#include "common.cuh"

namespace phx {
namespace {

// n mod d for any unsigned 64-bit n, with magic = floor((2^64 - 1) / d): the quotient estimate mulhi(n, magic)
// is at most 2 short, so two conditional subtractions finish the job.  (A 64-bit '%' by a run-time value costs
// ~100 instructions; this path made the gather instruction-bound.)
__device__ __forceinline__ unsigned long long umod_magic(unsigned long long n, unsigned long long d, unsigned long long magic) {
  unsigned long long r = n - __umul64hi(n, magic) * d;
  if (r >= d) r -= d;
  if (r >= d) r -= d;
  return r;
}
// raw = (id*scale + bias) mod M, floored (non-negative); idx = 0 if id == 0 else raw mod (buckets-1) + 1
__device__ __forceinline__ int hash_one(long long id, long long scale, long long bias, const HashFamilyDev& f) {
  if (id == 0) return 0;
  // wrapping int64 arithmetic, as numba / Rust release builds do
  const long long raw = (long long)((unsigned long long)id * (unsigned long long)scale + (unsigned long long)bias);
  const unsigned long long m = (unsigned long long)f.modulus;
  unsigned long long r;
  if (raw >= 0) r = umod_magic((unsigned long long)raw, m, f.magic_mod);
  else r = m - 1 - umod_magic((unsigned long long)(~raw), m, f.magic_mod);   // floored: -(x+1) mod m = m-1-(x mod m)
  return (int)umod_magic(r, (unsigned long long)f.buckets_m1, f.magic_bkt) + 1 + f.offset;
}

__device__ __forceinline__ void acc_row(float (&acc)[8], const bf16* row, int col) {
  uint4 u = __ldg(reinterpret_cast<const uint4*>(row + col));
  float2 a = unpack_bf2(u.x), b = unpack_bf2(u.y), c = unpack_bf2(u.z), d = unpack_bf2(u.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}

// The action row of a history token, columns col..col+7, as packed bf16.  Single action: row `act` of the table.
// Action set (multi_hot_to_embeddings, recsys_model.py:3282-3312): the [D] vector, the chunk these columns lie in
// signed by 2 a_v - 1 (a sign-bit flip: exact), everything zero when the set is empty.
__device__ __forceinline__ uint4 action_chunk(const TokenBuildArgs& a, int act, int col, bool action_set) {
  if (!action_set) return __ldg(reinterpret_cast<const uint4*>(a.action_table + (long long)act * a.D + col));
  const unsigned live = (a.num_action_types >= 32) ? 0xffffffffu : ((1u << a.num_action_types) - 1u);
  const unsigned bits = (unsigned)act & live;
  if (bits == 0u) return make_uint4(0u, 0u, 0u, 0u);
  uint4 u = __ldg(reinterpret_cast<const uint4*>(a.action_table + col));
  const int v = col / (a.D / a.num_action_types);
  if (!((bits >> v) & 1u)) { u.x ^= 0x80008000u; u.y ^= 0x80008000u; u.z ^= 0x80008000u; u.w ^= 0x80008000u; }
  return u;
}
__device__ __forceinline__ void acc_chunk(float (&acc)[8], uint4 u) {
  float2 a = unpack_bf2(u.x), b = unpack_bf2(u.y), c = unpack_bf2(u.z), d = unpack_bf2(u.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}

// One warp per token.  History token slots: post h0.., author h0.., action row, surface row;
// candidate token slots: post h0.., author h0...  x = bf16(bf16(sum) * input_scale).
// GENERAL = false is the benchmark's path with the optional inputs and outputs compiled out (packed rows, pre-hashed
// rows, landing buffer, projected tokens, action sets, fp32 rows, debug taps, rows-only): same arithmetic, fewer
// instructions in a kernel that is bound by how many loads it keeps in flight.
// Continuous history actions (project_continuous_value_to_embedding, recsys_model.py:1850-1886).  Hidden activations
// of every configured column for one token, gelu(norm(v) * w1), into hid[c][0..hidden): the warp's scratch.
__device__ __forceinline__ void cont_hidden(const TokenBuildArgs& a, const float* __restrict__ vals, int lane, float (*hid)[64]) {
  for (int c = 0; c < a.n_cont; ++c) {
    float v = __ldg(vals + a.cont_index[c]);
    v = fminf(fmaxf(v, 0.f), a.cont_scale[c]);                                        // normalize_continuous_value, 1756-1765
    v = a.cont_log[c] ? log1pf(v) / log1pf(a.cont_scale[c]) : v / a.cont_scale[c];
    for (int j = lane; j < a.cont_hidden; j += 32) hid[c][j] = gelu_tanh_f(v * __bfloat162float(a.cont_w1[c][j]));
  }
  __syncwarp();
}
// tv[0..8) (columns col..col+7 of the token, bf16-valued) += bf16(hid[c] @ w2[c]) for every configured column, one
// rounding per addend.
__device__ __forceinline__ void cont_add(const TokenBuildArgs& a, const float (*hid)[64], int col, float (&tv)[8]) {
  for (int c = 0; c < a.n_cont; ++c) {
    float e[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < a.cont_hidden; ++j) {
      const float h = hid[c][j];
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(a.cont_w2[c] + (long long)j * a.D + col));
      const float2 p0 = unpack_bf2(u.x), p1 = unpack_bf2(u.y), p2 = unpack_bf2(u.z), p3 = unpack_bf2(u.w);
      e[0] = fmaf(h, p0.x, e[0]); e[1] = fmaf(h, p0.y, e[1]); e[2] = fmaf(h, p1.x, e[2]); e[3] = fmaf(h, p1.y, e[3]);
      e[4] = fmaf(h, p2.x, e[4]); e[5] = fmaf(h, p2.y, e[5]); e[6] = fmaf(h, p3.x, e[6]); e[7] = fmaf(h, p3.y, e[7]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) tv[i] = round_bf(tv[i] + round_bf(e[i]));
  }
}

template <bool GENERAL>
__global__ void __launch_bounds__(256, GENERAL ? 3 : 5) build_tokens_kernel(TokenBuildArgs a) {
  // (no early launch signal here: the GEMM behind this kernel would park its CTAs - registers and all - on the SMs
  // while this bandwidth-bound kernel still needs every warp slot it can get)
  __shared__ float hid_s[GENERAL ? 8 : 1][PHX_MAX_HIST_CONT][64];
  const int T = a.S + a.C;
  const long long tok = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (tok >= (long long)a.B * T) return;
  // request and slot by 32-bit division (the launcher refuses B * T >= 2^31): a 64-bit '/' and '%' here cost more
  // instructions than the rest of the warp's prologue
  const int b = (int)((unsigned)tok / (unsigned)T), t = (int)((unsigned)tok - (unsigned)b * (unsigned)T);
  const int P = GENERAL ? a.P : 0;
  const bool is_front = t < a.S;              // rows in front of the candidates: user prefix + history
  const bool is_user = GENERAL && t < P;
  const bool is_hist = is_front && !is_user;
  const int Sh = a.S - P;                     // history slots of the input arrays
  const int H = a.item.num_hashes;
  const long long slot = is_user ? (long long)b : is_hist ? (long long)b * Sh + (t - P) : (long long)b * a.C + (t - a.S);
  long long orow;   // where this token's row goes
  if (GENERAL && a.pack.on() && !a.rows_only) {
    // packed rows: slots past the request's counts are not built at all (one token per warp: the whole warp leaves)
    if (is_front ? t >= a.pack.hist_cnt(b) : (t - a.S) >= a.pack.cand_cnt(b)) return;
    orow = is_front ? (long long)a.pack.hist_off[b] + t : a.pack.cand_base + a.pack.cand_off[b] + (t - a.S);
  } else {
    orow = token_row(a.split, a.B, a.S, T, b, t);
  }
  // lanes 0..H-1 hold the post rows, lanes H..2H-1 the author rows: hashed here, or taken as given; the user token
  // holds its user rows in lanes 0..Hu-1 and its IP rows behind them
  const int n_ip = (GENERAL && a.user_ip_hashes) ? a.Hip : 0;
  const int nrow = is_user ? a.Hu + n_ip : 2 * H;
  int my_idx = 0;
  if (is_user) {
    if (lane < a.Hu) my_idx = a.user_hashes[(long long)b * a.Hu + lane];
    else if (lane < nrow) my_idx = a.user_ip_hashes[(long long)b * a.Hip + (lane - a.Hu)];
  } else if (GENERAL && a.pre_hist_post) {
    if (lane < H) my_idx = (is_hist ? a.pre_hist_post : a.pre_cand_post)[slot * H + lane];
    else if (lane < 2 * H) my_idx = (is_hist ? a.pre_hist_author : a.pre_cand_author)[slot * H + (lane - H)];
  } else {
    const long long post_id = is_hist ? a.hist_post[slot] : a.cand_post[slot];
    const long long auth_id = is_hist ? a.hist_author[slot] : a.cand_author[slot];
    if (lane < H) my_idx = hash_one(post_id, a.item.scales[lane], a.item.biases[lane], a.item);
    else if (lane < 2 * H) {
      const int j = lane - H;
      my_idx = hash_one(auth_id, a.author.scales[j], a.author.biases[j], a.author);
    }
  }
  if (GENERAL && a.hashes && lane < 2 * H) a.hashes[tok * (2 * H) + lane] = my_idx;
  if (GENERAL && a.rows_only) return;   // uniform over the grid: the caller only wants the rows (exchange outside the kernel)
  const int first_hash = __shfl_sync(0xffffffffu, my_idx, 0);
  if (lane == 0) a.seg[orow] = (first_hash != 0) ? (is_front ? 1 : -1) : 0;
  int act = 0, srf = 0;
  if (is_hist) {
    if (GENERAL && a.hist_actions_bool) {   // the action set as the batch-prep hands it over: one byte per flag
      const unsigned char* f = a.hist_actions_bool + slot * a.num_action_types;
      act = (int)__ballot_sync(0xffffffffu, lane < a.num_action_types && f[lane] != 0);
    } else {
      act = a.hist_actions[slot];
    }
    srf = a.hist_surfaces[slot];
    if (!(GENERAL && a.action_multi_hot)) act = act < 0 ? 0 : (act > a.num_action_types ? a.num_action_types : act);
  } else if (GENERAL && !is_front && a.cand_surfaces) {
    srf = a.cand_surfaces[slot];
  }
  srf = srf < 0 ? 0 : (srf > a.num_surfaces ? a.num_surfaces : srf);
  const bool has_srf = is_hist || (GENERAL && !is_front && a.cand_surfaces);
  const bool has_cont = GENERAL && is_hist && a.n_cont > 0;
  float (*hid)[64] = hid_s[GENERAL ? (threadIdx.x >> 5) : 0];
  if (has_cont && !a.concat_hist) cont_hidden(a, a.hist_cont + slot * PHX_PREP_CONTINUOUS, lane, hid);
  // every lane takes part in these shuffles (lanes whose column chunk lies past D skip the loop below, so a
  // shuffle inside the loop would leave the warp split across two different shuffle instructions)
  const bf16* rowp[2 * PHX_MAX_HASHES];
  int my_pos = 0;   // exchanged rows: where slot `lane` of this token sits in the landing buffer
  if (GENERAL && a.landing && lane < 2 * H) my_pos = a.pos[tok * (2 * H) + lane];
#pragma unroll
  for (int j = 0; j < 2 * PHX_MAX_HASHES; ++j) {
    const int jj = j < nrow ? j : 0;
    const int idx = __shfl_sync(0xffffffffu, my_idx, jj);
    const int ps = __shfl_sync(0xffffffffu, my_pos, jj);
    rowp[j] = (GENERAL && a.landing) ? a.landing + (long long)ps * a.D : a.table.row_ptr(idx, a.D);
  }
  if (GENERAL && a.concat_hist) {
    // projected tokens: the gathered rows side by side - post rows, author rows, then the action and surface rows
    // (history) or the surface row (candidates that carry one); the user rows alone for the user token - as one GEMM
    // operand row (recsys_model.py:1903-1918, 2190-2221, 2307-2329); the projection, the addends, the scaling and
    // the row statistics follow in their own launches
    const int ngat = is_user ? a.Hu : 2 * H;
    const int nslot = ngat + (is_hist ? 2 : has_srf ? 1 : 0);
    bf16* dst = (is_user ? a.concat_user : is_hist ? a.concat_hist : a.concat_cand) + slot * (long long)nslot * a.D;
    for (int col = lane * 8; col < a.D; col += 256) {
#pragma unroll
      for (int j = 0; j < 2 * PHX_MAX_HASHES; ++j)
        if (j < ngat) *reinterpret_cast<uint4*>(dst + (long long)j * a.D + col) = __ldg(reinterpret_cast<const uint4*>(rowp[j] + col));
      if (is_hist)
        *reinterpret_cast<uint4*>(dst + (long long)ngat * a.D + col) = action_chunk(a, act, col, GENERAL && a.action_multi_hot);
      if (has_srf)
        *reinterpret_cast<uint4*>(dst + (long long)(nslot - 1) * a.D + col) =
            __ldg(reinterpret_cast<const uint4*>(a.surface_table + (long long)srf * a.D + col));
    }
    return;
  }
  float row_ss = 0.f;
  for (int col = lane * 8; col < a.D; col += 256) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2 * PHX_MAX_HASHES; ++j)
      if (j < nrow) acc_row(acc, rowp[j], col);
    if (is_hist) acc_chunk(acc, action_chunk(a, act, col, GENERAL && a.action_multi_hot));
    if (has_srf) acc_row(acc, a.surface_table + (long long)srf * a.D, col);
    float tv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) tv[i] = round_bf(acc[i]);
    if (has_cont) cont_add(a, hid, col, tv);
    uint4 o;
    if (GENERAL && a.tokens) {
      o.x = pack_bf2(tv[0], tv[1]); o.y = pack_bf2(tv[2], tv[3]); o.z = pack_bf2(tv[4], tv[5]); o.w = pack_bf2(tv[6], tv[7]);
      *reinterpret_cast<uint4*>(a.tokens + tok * a.D + col) = o;
    }
    if (GENERAL && a.x32) {   // full-precision path: the token is the bf16 sum, its scaled value stays fp32
      float* dst = a.x32 + orow * a.D + col;
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[i] = tv[i] * a.input_scale;
      continue;
    }
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i] = round_bf(tv[i] * a.input_scale); row_ss += s[i] * s[i]; }
    o.x = pack_bf2(s[0], s[1]); o.y = pack_bf2(s[2], s[3]); o.z = pack_bf2(s[4], s[5]); o.w = pack_bf2(s[6], s[7]);
    *reinterpret_cast<uint4*>(a.x + orow * a.D + col) = o;
  }
  if (a.row_ss) {   // statistics of the bf16 row for the first fused RMSNorm
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) row_ss += __shfl_xor_sync(0xffffffffu, row_ss, o);
    if (lane < a.ss_slots) a.row_ss[orow * a.ss_slots + lane] = (lane == 0) ? row_ss : 0.f;
  }
}

// Projected tokens, last step: x = bf16(token * input_scale) at the token's row of the residual stream (plain or
// split layout) with the row statistics of the first fused RMSNorm; tok_user [B, D], tok_hist [B*(S-P), D] and
// tok_cand [B*C, D] are the outputs of the projection GEMMs.  The addends of the reference's blocks that follow their
// projection are applied here: the sum of the IP rows on the user token (recsys_model.py:1920-1923) and the
// continuous-action embeddings on the history tokens (2249-2271).  One warp per token.
__global__ void __launch_bounds__(256) finish_tokens_kernel(const bf16* __restrict__ tok_user, const bf16* __restrict__ tok_hist,
                                                            const bf16* __restrict__ tok_cand, TokenBuildArgs a) {
  __shared__ float hid_s[8][PHX_MAX_HIST_CONT][64];
  const int T = a.S + a.C;
  const long long tok = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (tok >= (long long)a.B * T) return;
  // request and slot by 32-bit division (the launcher refuses B * T >= 2^31): a 64-bit '/' and '%' here cost more
  // instructions than the rest of the warp's prologue
  const int b = (int)((unsigned)tok / (unsigned)T), t = (int)((unsigned)tok - (unsigned)b * (unsigned)T);
  const int Sh = a.S - a.P;
  const bool is_user = t < a.P, is_hist = !is_user && t < a.S;
  const bf16* src = is_user ? tok_user + (long long)b * a.D
                  : is_hist ? tok_hist + ((long long)b * Sh + (t - a.P)) * a.D : tok_cand + ((long long)b * a.C + (t - a.S)) * a.D;
  long long orow;
  if (a.pack.on()) {
    if (t < a.S ? t >= a.pack.hist_cnt(b) : (t - a.S) >= a.pack.cand_cnt(b)) return;
    orow = t < a.S ? (long long)a.pack.hist_off[b] + t : a.pack.cand_base + a.pack.cand_off[b] + (t - a.S);
  } else {
    orow = token_row(a.split, a.B, a.S, T, b, t);
  }
  const bool has_cont = is_hist && a.n_cont > 0;
  const int n_ip = (is_user && a.user_ip_hashes) ? a.Hip : 0;
  float (*hid)[64] = hid_s[threadIdx.x >> 5];
  if (has_cont) cont_hidden(a, a.hist_cont + ((long long)b * Sh + (t - a.P)) * PHX_PREP_CONTINUOUS, lane, hid);
  float row_ss = 0.f;
  for (int col = lane * 8; col < a.D; col += 256) {
    uint4 u = *reinterpret_cast<const uint4*>(src + col);
    const float2 p0 = unpack_bf2(u.x), p1 = unpack_bf2(u.y), p2 = unpack_bf2(u.z), p3 = unpack_bf2(u.w);
    float s[8] = {p0.x, p0.y, p1.x, p1.y, p2.x, p2.y, p3.x, p3.y};
    if (n_ip > 0) {
      float ip[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < n_ip; ++j) acc_row(ip, a.table.row_ptr(__ldg(a.user_ip_hashes + (long long)b * a.Hip + j), a.D), col);
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i] = round_bf(s[i] + round_bf(ip[i]));
    }
    if (has_cont) cont_add(a, hid, col, s);
    if (n_ip > 0 || has_cont) { u.x = pack_bf2(s[0], s[1]); u.y = pack_bf2(s[2], s[3]); u.z = pack_bf2(s[4], s[5]); u.w = pack_bf2(s[6], s[7]); }
    if (a.tokens) *reinterpret_cast<uint4*>(a.tokens + tok * a.D + col) = u;
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i] = round_bf(s[i] * a.input_scale); row_ss += s[i] * s[i]; }
    uint4 o;
    o.x = pack_bf2(s[0], s[1]); o.y = pack_bf2(s[2], s[3]); o.z = pack_bf2(s[4], s[5]); o.w = pack_bf2(s[6], s[7]);
    *reinterpret_cast<uint4*>(a.x + orow * a.D + col) = o;
  }
  if (a.row_ss) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) row_ss += __shfl_xor_sync(0xffffffffu, row_ss, o);
    if (lane < a.ss_slots) a.row_ss[orow * a.ss_slots + lane] = (lane == 0) ? row_ss : 0.f;
  }
}

// Packed rows: the position of every packed row (RoPE) and, for the candidate rows, the slot of the [B, C] output
// arrays each one answers.  One thread per (request, slot).
__global__ void pack_plan_kernel(PackMap pk, int B, int S, int C, int* __restrict__ pos_rows, int* __restrict__ out_index) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int T = S + C;
  if (i >= (long long)B * T) return;
  const int b = (int)(i / T), t = (int)(i % T);
  if (t < S) {
    if (t < pk.hist_cnt(b)) pos_rows[pk.hist_off[b] + t] = t;
  } else if (t - S < pk.cand_cnt(b)) {
    const int r = pk.cand_off[b] + (t - S);
    pos_rows[pk.cand_base + r] = S;               // every candidate sits at the first position after the history
    out_index[r] = b * C + (t - S);
  }
}

__global__ void hash_ids_kernel(HashFamilyDev fam, const long long* __restrict__ ids, long long n, int* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * fam.num_hashes) return;
  const long long t = i / fam.num_hashes;
  const int j = (int)(i % fam.num_hashes);
  out[i] = hash_one(ids[t], fam.scales[j], fam.biases[j], fam);
}

// Stand-alone gather-sum: out[i] = bf16(sum_j table[hash_j(id_i)]) in hash order.  LANES lanes per id
// (LANES * 8 >= D or a loop), several ids per warp for narrow rows.
template <int LANES>
__global__ void __launch_bounds__(256) gather_sum_kernel(HashFamilyDev fam, TableView table, int D,
                                                         const long long* __restrict__ ids,
                                                         long long n, bf16* __restrict__ out) {
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LANES;
  const int sub = threadIdx.x % LANES;
  const bool valid = gid < n;   // no early return: the shuffles below need every lane of the warp
  const long long id = valid ? __ldg(ids + gid) : 0;
  // lane j of the id's lane group computes hash j; the group shares the results by shuffle
  int mine = 0;
  if (sub < fam.num_hashes) {
    mine = hash_one(id, fam.scales[sub], fam.biases[sub], fam);
  }
  const bf16* rowp[PHX_MAX_HASHES];
#pragma unroll
  for (int j = 0; j < PHX_MAX_HASHES; ++j) rowp[j] = table.row_ptr(__shfl_sync(0xffffffffu, mine, j, LANES), D);
  for (int col = sub * 8; col < D && valid; col += LANES * 8) {
    uint4 u[PHX_MAX_HASHES];
#pragma unroll
    for (int j = 0; j < PHX_MAX_HASHES; ++j)
      if (j < fam.num_hashes) u[j] = __ldg(reinterpret_cast<const uint4*>(rowp[j] + col));
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < PHX_MAX_HASHES; ++j) {
      if (j < fam.num_hashes) {
        float2 a = unpack_bf2(u[j].x), b = unpack_bf2(u[j].y), c = unpack_bf2(u[j].z), d = unpack_bf2(u[j].w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
        acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
      }
    }
    uint4 o;
    o.x = pack_bf2(acc[0], acc[1]); o.y = pack_bf2(acc[2], acc[3]); o.z = pack_bf2(acc[4], acc[5]); o.w = pack_bf2(acc[6], acc[7]);
    __stcs(reinterpret_cast<uint4*>(out + gid * D + col), o);
  }
}

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float synth_value(unsigned long long row, int col, int width, uint32_t seed, float scale) {
  uint32_t x = (uint32_t)((row * (unsigned long long)width + (unsigned long long)col) & 0xFFFFFFFFull) ^ seed;
  x = mix32(x);
  return ((float)(x >> 16) - 32768.0f) * scale;
}

__global__ void table_fill_kernel(bf16* table, long long row0, long long rows, int width, uint32_t seed, float scale) {
  const long long total = rows * (long long)(width / 8);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (width / 8);
    const int c = (int)(i % (width / 8)) * 8;
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = synth_value((unsigned long long)(row0 + r), c + k, width, seed, scale);
    uint4 o;
    o.x = pack_bf2(v[0], v[1]); o.y = pack_bf2(v[2], v[3]); o.z = pack_bf2(v[4], v[5]); o.w = pack_bf2(v[6], v[7]);
    *reinterpret_cast<uint4*>(table + r * width + c) = o;
  }
}

// corpus rows: synthetic values rounded to bf16, fixed-order fp32 sum of squares, scaled, rounded again
__global__ void corpus_fill_kernel(bf16* rows_ptr, long long global_row0, long long rows, int dim, uint32_t seed) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int c = 0; c < dim; ++c) {
      float v = round_bf(synth_value((unsigned long long)(global_row0 + r), c, dim, seed, 1.0f / 32768.0f));
      acc = acc + v * v;
    }
    const float inv = 1.0f / sqrtf(fmaxf(acc, 1e-12f));
    for (int c = 0; c < dim; c += 8) {
      float v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        v[k] = round_bf(synth_value((unsigned long long)(global_row0 + r), c + k, dim, seed, 1.0f / 32768.0f)) * inv;
      uint4 o;
      o.x = pack_bf2(v[0], v[1]); o.y = pack_bf2(v[2], v[3]); o.z = pack_bf2(v[4], v[5]); o.w = pack_bf2(v[6], v[7]);
      *reinterpret_cast<uint4*>(rows_ptr + r * dim + c) = o;
    }
  }
}

}  // namespace

phx_status build_tokens_launch(const TokenBuildArgs& a, cudaStream_t stream, std::string& err) {
  if (a.D % 8 != 0 || a.item.num_hashes != a.author.num_hashes || 2 * a.item.num_hashes > 32) {
    err = "build_tokens: D must be a multiple of 8 and hash counts must match";
    return PHX_E_ARG;
  }
  const long long toks = (long long)a.B * (a.S + a.C);
  if (toks == 0) return PHX_OK;
  if (toks >= (1ll << 31)) { err = "build_tokens: more than 2^31 tokens in one call"; return PHX_E_CAPACITY; }
  const int warps = 8;
  const bool general = a.pack.hist_off || a.pre_hist_post || a.landing || a.concat_hist || a.action_multi_hot || a.x32 ||
                       a.tokens || a.hashes || a.rows_only || a.P || a.hist_actions_bool || a.cand_surfaces || a.n_cont;
  if (a.P && (a.Hu <= 0 || a.Hu + a.Hip > 2 * PHX_MAX_HASHES || !a.user_hashes)) { err = "build_tokens: user-prefix arguments"; return PHX_E_ARG; }
  if (a.n_cont && (a.cont_hidden <= 0 || a.cont_hidden > 64 || !a.hist_cont)) { err = "build_tokens: continuous-action arguments"; return PHX_E_ARG; }
  if (general) build_tokens_kernel<true><<<(unsigned)((toks + warps - 1) / warps), warps * 32, 0, stream>>>(a);
  else build_tokens_kernel<false><<<(unsigned)((toks + warps - 1) / warps), warps * 32, 0, stream>>>(a);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status pack_plan_launch(const PackMap& pk, int B, int S, int C, int* pos_rows, int* out_index, cudaStream_t stream,
                            std::string& err) {
  const long long n = (long long)B * (S + C);
  if (n == 0) return PHX_OK;
  pack_plan_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(pk, B, S, C, pos_rows, out_index);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status finish_tokens_launch(const bf16* tok_user, const bf16* tok_hist, const bf16* tok_cand, const TokenBuildArgs& a,
                                cudaStream_t stream, std::string& err) {
  const long long toks = (long long)a.B * (a.S + a.C);
  if (toks == 0) return PHX_OK;
  if (toks >= (1ll << 31)) { err = "finish_tokens: more than 2^31 tokens in one call"; return PHX_E_CAPACITY; }
  finish_tokens_kernel<<<(unsigned)((toks + 7) / 8), 256, 0, stream>>>(tok_user, tok_hist, tok_cand, a);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status hash_ids_launch(const HashFamilyDev& fam, const long long* ids, long long n, int* out, cudaStream_t stream,
                           std::string& err) {
  const long long total = n * fam.num_hashes;
  if (total == 0) return PHX_OK;
  hash_ids_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(fam, ids, n, out);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status gather_sum_launch(const HashFamilyDev& fam, const TableView& table, int D,
                             const long long* ids, long long n, bf16* out, cudaStream_t stream, std::string& err) {
  if (D % 8 != 0) { err = "gather_sum: D must be a multiple of 8"; return PHX_E_ARG; }
  if (n == 0) return PHX_OK;
  if (D <= 128) {
    gather_sum_kernel<16><<<(unsigned)((n * 16 + 255) / 256), 256, 0, stream>>>(fam, table, D, ids, n, out);
  } else {
    gather_sum_kernel<32><<<(unsigned)((n * 32 + 255) / 256), 256, 0, stream>>>(fam, table, D, ids, n, out);
  }
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status table_fill_launch(bf16* table, long long row0, long long rows, int width, uint32_t seed, float amp,
                             cudaStream_t stream, std::string& err) {
  if (rows == 0) return PHX_OK;
  table_fill_kernel<<<148 * 8, 256, 0, stream>>>(table, row0, rows, width, seed, amp / 32768.0f);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status corpus_fill_launch(bf16* rows_ptr, long long global_row0, long long rows, int dim, uint32_t seed,
                              cudaStream_t stream, std::string& err) {
  if (rows == 0) return PHX_OK;
  corpus_fill_kernel<<<148 * 8, 256, 0, stream>>>(rows_ptr, global_row0, rows, dim, seed);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

}  // namespace phx
