// The value model behind the heads (xai-value-model/scoring.rs): fuse_heads with its per-candidate gates and the
// multiplicative mode (67-261), the request's user_video_continuation (263-280), exploration bonus (491-496),
// cold-start lift (414-431), author diversity (304-327, 368-402), out-of-network weight (329-338) and class factors
// (340-366), all in f64 and in the reference's operation order.  One thread block per request; the two steps that
// the reference does by sorting (rank of a candidate among its author's candidates, the score at a given rank) are
// done by counting the candidates that come before in (score descending, input order) - the order a stable sort
// gives - so nothing is sorted.  The work is a few hundred f64 operations per candidate: latency, not throughput,
// is what matters, and it rides on the stream right behind the heads kernel.
#include <math.h>

#include "common.cuh"

namespace phx {
namespace {

constexpr double VM_OFFSET = 0.001;                 // NEGATIVE_SCORES_OFFSET, weights.rs:4
constexpr double VM_MIN_POWER_OFFSET = 1e-2;        // weights.rs:5
constexpr double VM_MIN_SKIP_BASE = 1e-6;           // scoring.rs:4

// index of each PhoenixScores field in phx_value_model.src
enum VmField { F_FAVORITE = 0, F_REPLY, F_RETWEET, F_PHOTO_EXPAND, F_VIDEO_OPEN, F_CLICK, F_OPEN_LINK, F_PROFILE_CLICK, F_VQV,
               F_SHARE, F_SHARE_DM, F_SHARE_LINK, F_DWELL, F_QUOTE, F_QUOTED_CLICK, F_QUOTED_VQV, F_FOLLOW_AUTHOR,
               F_NOT_INTERESTED, F_BLOCK_AUTHOR, F_MUTE_AUTHOR, F_REPORT, F_NOT_DWELLED, F_POST_UNEXPLORED, F_POST_VIDEO,
               F_GROK_ANALYZE, F_DWELL_TIME, F_CLICK_DWELL_TIME, F_HOME_VIDEO_CONT, F_HOME_PROFILE_VISIT };
// index of each term of weighted_terms (scoring.rs:145-260) in phx_value_model.w
enum VmTerm { T_FAVORITE = 0, T_REPLY, T_RETWEET, T_PHOTO_EXPAND, T_VIDEO_OPEN, T_CLICK, T_OPEN_LINK, T_PROFILE_CLICK, T_VQV,
              T_SHARE, T_SHARE_DM, T_SHARE_LINK, T_DWELL, T_QUOTE, T_QUOTED_CLICK, T_QUOTED_VQV, T_DWELL_TIME,
              T_CLICK_DWELL_TIME, T_VIDEO_CONT, T_USER_VIDEO_CONT, T_PROFILE_VISIT, T_FOLLOW_AUTHOR, T_NOT_INTERESTED,
              T_BLOCK_AUTHOR, T_MUTE_AUTHOR, T_REPORT, T_NOT_DWELLED, T_POST_UNEXPLORED, T_POST_VIDEO, T_GROK_ANALYZE };

struct Opt { double v; bool some; };   // Option<f64>

// the candidate's value of one PhoenixScores field
__device__ __forceinline__ Opt field(const phx_value_model& m, const phx_value_inputs& in, long long cand, int f) {
  const int s = m.src[f];
  if (s < 0) return {0.0, false};
  if (s < in.num_actions) return {exp((double)in.log_probs[cand * in.num_actions + s]), true};
  return {(double)in.continuous[cand * in.num_continuous + (s - in.num_actions)], true};
}
__device__ __forceinline__ double apply(Opt s, double w) { return (s.some ? s.v : 0.0) * w; }          // scoring.rs:59-61
__device__ __forceinline__ Opt product(Opt a, Opt b) { return {a.v * b.v, a.some && b.some}; }         // 63-65

__device__ __forceinline__ double offset_score(double s, const phx_value_model& m) {                   // 282-291
  if (m.offset_total_sum == 0.0) return fmax(s, 0.0);
  if (s < 0.0) return (s + m.offset_negative_sum) / m.offset_total_sum * VM_OFFSET;
  return s + VM_OFFSET;
}
__device__ __forceinline__ double unoffset_score(double w, const phx_value_model& m) {                 // 293-302
  if (m.offset_total_sum == 0.0) return w;
  if (w < VM_OFFSET) return w / VM_OFFSET * m.offset_total_sum - m.offset_negative_sum;
  return w - VM_OFFSET;
}

// weighted_terms (scoring.rs:122-261) into t[30], in the reference's order
__device__ void weighted_terms(const phx_value_model& m, const phx_value_inputs& in, long long cand, unsigned flags, Opt user_cont,
                               double (&t)[PHX_VM_TERMS]) {
  const bool in_net = (flags & PHX_VM_IN_NETWORK_KNOWN) && (flags & PHX_VM_IN_NETWORK);
  const bool boost_ok = !(flags & PHX_VM_IS_REPLY) && !(flags & PHX_VM_IS_RETWEET) && (flags & PHX_VM_MUTUAL_FOLLOW);   // inputs.rs:19-23
  const double vqv_w = (flags & PHX_VM_VQV_ELIGIBLE) ? m.w[T_VQV] : 0.0;
  const double qvqv_w = (flags & PHX_VM_QUOTED_VQV_ELIGIBLE) ? m.w[T_QUOTED_VQV] : 0.0;
  const double unexpl_w = (m.post_unexplored_include_oon || in_net) ? m.w[T_POST_UNEXPLORED] : 0.0;
  const double reply_w = (m.reply_boost != 0.0 && boost_ok) ? m.w[T_REPLY] + m.reply_boost : m.w[T_REPLY];   // weights.rs:131-139
  const double dwell_w = (m.dwell_boost != 0.0 && boost_ok) ? m.w[T_DWELL] + m.dwell_boost : m.w[T_DWELL];   // 141-149
  auto f = [&](int which) { return field(m, in, cand, which); };
  const Opt video_open = f(F_VIDEO_OPEN), profile_click = f(F_PROFILE_CLICK);
  t[T_FAVORITE] = apply(f(F_FAVORITE), m.w[T_FAVORITE]);
  t[T_REPLY] = apply(f(F_REPLY), reply_w);
  t[T_RETWEET] = apply(f(F_RETWEET), m.w[T_RETWEET]);
  t[T_PHOTO_EXPAND] = apply(f(F_PHOTO_EXPAND), m.w[T_PHOTO_EXPAND]);
  t[T_VIDEO_OPEN] = apply(video_open, m.w[T_VIDEO_OPEN]);
  t[T_CLICK] = apply(f(F_CLICK), m.w[T_CLICK]);
  t[T_OPEN_LINK] = apply(f(F_OPEN_LINK), m.w[T_OPEN_LINK]);
  t[T_PROFILE_CLICK] = apply(profile_click, m.w[T_PROFILE_CLICK]);
  t[T_VQV] = apply(f(F_VQV), vqv_w);
  t[T_SHARE] = apply(f(F_SHARE), m.w[T_SHARE]);
  t[T_SHARE_DM] = apply(f(F_SHARE_DM), m.w[T_SHARE_DM]);
  t[T_SHARE_LINK] = apply(f(F_SHARE_LINK), m.w[T_SHARE_LINK]);
  t[T_DWELL] = apply(f(F_DWELL), dwell_w);
  t[T_QUOTE] = apply(f(F_QUOTE), m.w[T_QUOTE]);
  t[T_QUOTED_CLICK] = apply(f(F_QUOTED_CLICK), m.w[T_QUOTED_CLICK]);
  t[T_QUOTED_VQV] = apply(f(F_QUOTED_VQV), qvqv_w);
  t[T_DWELL_TIME] = apply(f(F_DWELL_TIME), m.w[T_DWELL_TIME]);
  t[T_CLICK_DWELL_TIME] = apply(f(F_CLICK_DWELL_TIME), m.w[T_CLICK_DWELL_TIME]);
  t[T_VIDEO_CONT] = apply(product(video_open, f(F_HOME_VIDEO_CONT)), m.w[T_VIDEO_CONT]);
  t[T_USER_VIDEO_CONT] = apply(product(video_open, user_cont), m.w[T_USER_VIDEO_CONT]);
  t[T_PROFILE_VISIT] = apply(product(profile_click, f(F_HOME_PROFILE_VISIT)), m.w[T_PROFILE_VISIT]);
  t[T_FOLLOW_AUTHOR] = apply(f(F_FOLLOW_AUTHOR), m.w[T_FOLLOW_AUTHOR]);
  t[T_NOT_INTERESTED] = apply(f(F_NOT_INTERESTED), m.w[T_NOT_INTERESTED]);
  t[T_BLOCK_AUTHOR] = apply(f(F_BLOCK_AUTHOR), m.w[T_BLOCK_AUTHOR]);
  t[T_MUTE_AUTHOR] = apply(f(F_MUTE_AUTHOR), m.w[T_MUTE_AUTHOR]);
  t[T_REPORT] = apply(f(F_REPORT), m.w[T_REPORT]);
  t[T_NOT_DWELLED] = apply(f(F_NOT_DWELLED), m.w[T_NOT_DWELLED]);
  t[T_POST_UNEXPLORED] = apply(f(F_POST_UNEXPLORED), unexpl_w);
  t[T_POST_VIDEO] = apply(f(F_POST_VIDEO), m.w[T_POST_VIDEO]);
  t[T_GROK_ANALYZE] = apply(f(F_GROK_ANALYZE), m.w[T_GROK_ANALYZE]);
}

// fuse_heads (scoring.rs:67-110)
__device__ double fuse_heads(const phx_value_model& m, const phx_value_inputs& in, long long cand, unsigned flags, Opt user_cont) {
  double t[PHX_VM_TERMS];
  weighted_terms(m, in, cand, flags, user_cont, t);
  if (!m.multiplicative) {
    double s = 0.0;
#pragma unroll 1
    for (int i = 0; i < PHX_VM_TERMS; ++i) s = s + t[i];   // compute_weighted_score: left to right
    return offset_score(s, m);
  }
  double engage = 0.0;                                      // engage_sum: all terms but dwell_time and not_dwelled
#pragma unroll 1
  for (int i = 0; i < PHX_VM_TERMS; ++i)
    if (i != T_DWELL_TIME && i != T_NOT_DWELLED) engage = engage + t[i];
  engage = engage + m.engage_bias;
  if (engage < 0.0) return offset_score(engage, m);
  double skip = 1.0;                                        // skip_score
  const Opt p = field(m, in, cand, F_NOT_DWELLED);
  if (p.some && isfinite(p.v) && m.not_dwelled_power_exponent != 0.0)
    skip = pow(fmax(p.v + fmax(m.not_dwelled_power_offset, VM_MIN_POWER_OFFSET), VM_MIN_SKIP_BASE), m.not_dwelled_power_exponent);
  const double time_factor = 1.0 + fmax(apply(field(m, in, cand, F_DWELL_TIME), m.w[T_DWELL_TIME]), 0.0);
  return offset_score(skip * engage * time_factor, m);
}

// candidates that a stable sort by score, highest first, puts in front of candidate i (all of them, or only those of
// i's author)
__device__ __forceinline__ int count_before(const double* s, const long long* author, int n, int i, bool same_author_only) {
  const double si = s[i];
  const long long ai = author[i];
  int k = 0;
  for (int j = 0; j < n; ++j) {
    const bool before = s[j] > si || (s[j] == si && j < i);
    k += (before && (!same_author_only || author[j] == ai)) ? 1 : 0;
  }
  return k;
}

__device__ __forceinline__ bool oon_applies(const phx_value_model& m, unsigned flags) {                // scoring.rs:329-338
  if (!(flags & PHX_VM_IN_NETWORK_KNOWN)) return false;
  if (!(flags & PHX_VM_IN_NETWORK)) return true;
  return m.oon_rescore_in_network_replies_retweets && (flags & (PHX_VM_IS_REPLY | PHX_VM_IS_RETWEET));
}

__global__ void __launch_bounds__(256) value_scores_kernel(phx_value_model m, phx_value_inputs in, double* weighted_out,
                                                           double* scores_out) {
  extern __shared__ double vsm[];
  const int C = in.num_candidates;
  double* s_ord = vsm;                                          // ordering scores of the current stage
  double* s_w = vsm + C;                                        // weighted scores
  long long* s_auth = reinterpret_cast<long long*>(vsm + 2 * C);
  __shared__ double sh_user_cont, sh_lift_val;
  __shared__ int sh_user_some, sh_lift_idx;
  const int b = blockIdx.x;
  const long long base = (long long)b * C;
  int n = in.num_valid ? in.num_valid[b] : C;
  n = n < 0 ? 0 : (n > C ? C : n);
  double eow = 1.0, oon_f[2] = {0.0, 0.0}, inn_f[2] = {0.0, 0.0};
  bool oon_some = false, inn_some = false;
  if (in.context) {
    const double* cx = in.context + (long long)b * 5;
    eow = cx[0];
    oon_some = !isnan(cx[1]); oon_f[0] = cx[1]; oon_f[1] = cx[2];
    inn_some = !isnan(cx[3]); inn_f[0] = cx[3]; inn_f[1] = cx[4];
  }
  const bool cached = in.weighted != nullptr && !m.multiplicative;                                    // scoring.rs:445-450
  // set_user_video_continuation (263-280): two left-to-right folds over the request's candidates.  The products are
  // formed by all threads, the two sums run in candidate order on one thread (a candidate that lacks either value
  // adds nothing, here as 0.0).
  const bool want_user_cont = !cached && m.src[F_VIDEO_OPEN] >= 0 && m.src[F_HOME_VIDEO_CONT] >= 0 && m.w[T_USER_VIDEO_CONT] != 0.0;
  if (want_user_cont) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const Opt o = field(m, in, base + i, F_VIDEO_OPEN), c = field(m, in, base + i, F_HOME_VIDEO_CONT);
      s_ord[i] = o.v * c.v;
      s_w[i] = o.v;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    sh_lift_idx = 0x7fffffff;
    sh_lift_val = 0.0;
    double secs = 0.0, opens = 0.0;
    if (want_user_cont)
      for (int i = 0; i < n; ++i) { secs = secs + s_ord[i]; opens = opens + s_w[i]; }
    sh_user_some = opens > 0.0;
    sh_user_cont = opens > 0.0 ? secs / opens : 0.0;
  }
  __syncthreads();
  const Opt user_cont = {sh_user_cont, sh_user_some != 0};
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const unsigned fl = in.flags ? in.flags[base + i] : 0u;
    const double w = cached ? in.weighted[base + i] : fuse_heads(m, in, base + i, fl, user_cont);
    s_w[i] = w;
    s_auth[i] = in.author_ids ? in.author_ids[base + i] : 0;
    if (weighted_out) weighted_out[base + i] = w;
    if (in.cold_start_rank && in.cold_start_rank[base + i] >= 0) atomicMin(&sh_lift_idx, i);          // first candidate with a lift
  }
  __syncthreads();
  const int lift_idx = sh_lift_idx;
  const int lift_rank = lift_idx < n ? in.cold_start_rank[base + lift_idx] : -1;
  const bool lift = lift_rank >= 0 && lift_rank < n;                                                  // scoring.rs:421-423
  auto diversity = [&](const double* ord, int i) {                                                    // 304-327, 374-387
    if (!m.enable_author_diversity) return 1.0;
    const int k = count_before(ord, s_auth, n, i, true);
    return (1.0 - m.author_diversity_floor) * pow(m.author_diversity_decay, (double)k) + m.author_diversity_floor;
  };
  // apply_cold_start_decisions (414-431) on s_ord: the lifted candidate gets at least the score at its target rank
  auto cold_start = [&]() {
    if (!lift) return;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      if (count_before(s_ord, s_auth, n, i, false) == lift_rank) sh_lift_val = s_ord[i];
    __syncthreads();
    if (threadIdx.x == 0) s_ord[lift_idx] = fmax(s_ord[lift_idx], sh_lift_val);
    __syncthreads();
  };
  if (m.multiplier_pre_offset) {                                                                      // 452-467
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const unsigned fl = in.flags ? in.flags[base + i] : 0u;
      const double ad = diversity(s_w, i);
      const double oon = oon_applies(m, fl) ? eow : 1.0;
      const double net = unoffset_score(s_w[i], m) + (in.exploration_bonus ? in.exploration_bonus[base + i] : 0.0);
      const double scaled = net >= 0.0 ? (ad * oon) * net : net;
      s_ord[i] = offset_score(scaled, m);
    }
    __syncthreads();
    cold_start();
    for (int i = threadIdx.x; i < n; i += blockDim.x) scores_out[base + i] = s_ord[i];
    return;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {                                                 // 469-473, 491-496
    const double bonus = in.exploration_bonus ? in.exploration_bonus[base + i] : 0.0;
    s_ord[i] = bonus == 0.0 ? s_w[i] : offset_score(unoffset_score(s_w[i], m) + bonus, m);
  }
  __syncthreads();
  cold_start();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {                                                 // 475-488
    const unsigned fl = in.flags ? in.flags[base + i] : 0u;
    const double s = s_ord[i];
    const double ad = diversity(s_ord, i);
    const double oon = oon_applies(m, fl) ? eow : 1.0;
    // class_factor_score (340-366)
    bool cs_some = false;
    double cs = 0.0;
    if (!m.multiplicative && (fl & PHX_VM_IN_NETWORK_KNOWN)) {
      const bool in_net = (fl & PHX_VM_IN_NETWORK) != 0;
      const bool have = in_net ? inn_some : oon_some;
      if (have) {
        const double* fac = in_net ? inn_f : oon_f;
        const double level = in_net ? oon : 1.0;
        double dwell = apply(field(m, in, base + i, F_DWELL_TIME), m.w[T_DWELL_TIME]);
        dwell = (s >= VM_OFFSET && isfinite(dwell)) ? fmin(fmax(dwell, 0.0), s) : 0.0;
        cs = level * (fac[0] * (s - dwell) + fac[1] * dwell);
        cs_some = true;
      }
    }
    scores_out[base + i] = cs_some ? cs * ad : s * ad * oon;
  }
}

}  // namespace
}  // namespace phx

extern "C" phx_status phx_value_scores_device(int32_t device, const phx_value_model* model, const phx_value_inputs* in,
                                              double* weighted_out, double* scores_out, void* stream) {
  using namespace phx;
  std::string err;
  auto fail = [&](phx_status st, const char* msg) { set_global_error(msg); return st; };
  if (!model || !in || !scores_out) return fail(PHX_E_ARG, "phx_value_scores_device: null argument");
  if (in->batch < 0 || in->num_candidates <= 0 || in->num_actions < 0 || in->num_continuous < 0)
    return fail(PHX_E_ARG, "phx_value_scores_device: sizes");
  if (in->num_candidates > PHX_VM_MAX_CANDIDATES) return fail(PHX_E_CAPACITY, "phx_value_scores_device: more than 4096 candidates per request");
  for (int f = 0; f < PHX_VM_FIELDS; ++f) {
    const int s = model->src[f];
    if (s >= in->num_actions + in->num_continuous) return fail(PHX_E_ARG, "phx_value_scores_device: source column out of range");
    if (s >= 0 && s < in->num_actions && !in->log_probs) return fail(PHX_E_ARG, "phx_value_scores_device: log_probs missing");
    if (s >= in->num_actions && !in->continuous) return fail(PHX_E_ARG, "phx_value_scores_device: continuous missing");
  }
  if (in->batch == 0) return PHX_OK;
  if (cudaSetDevice(device) != cudaSuccess) return fail(PHX_E_CUDA, "cudaSetDevice failed");
  const size_t smem = (size_t)in->num_candidates * 24;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(value_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return fail(PHX_E_CUDA, "phx_value_scores_device: shared memory attribute");
  }
  value_scores_kernel<<<in->batch, 256, smem, (cudaStream_t)stream>>>(*model, *in, weighted_out, scores_out);
  const cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(PHX_E_CUDA, cudaGetErrorString(ce));
  return PHX_OK;
}
