// Diversity rerank behind the value model: greedy DPP selection and its sliding-window variant for a batch of requests,
// one thread block per request (vm-ranker/dpp.rs:45-413).  f64 throughout, operations in the reference's order: the
// kernel L_ij = q_i q_j cos_ij over the top `max_selected_rank` candidates by score (plus a pinned seed), greedy MAP by
// incremental Cholesky (first item of largest conditional variance wins a tie), served in score order or pick order.
// The dot product is the reference's scalar definition (each product in f32, the sum in f64, vm-ranker/helpers.rs:
// 21-28).  Where the reference's unstable sort leaves equal scores in unspecified order, the lower input index goes
// first.
#include <cuda_fp16.h>
#include <math.h>
#include <string.h>

#include <string>

#include "common.cuh"

namespace phx {
namespace {

constexpr int DPP_THREADS = 256;
constexpr double DPP_EPS = 1e-6;

struct DppKernelArgs {
  phx_dpp_config cfg;
  phx_dpp_inputs in;
  int* out_index; double* out_score; int* out_count;
};

__device__ __forceinline__ double dpp_dot(const __half* a, const __half* b, int E) {
  double acc = 0.0;
  for (int e = 0; e < E; ++e) acc += (double)(__half2float(a[e]) * __half2float(b[e]));
  return acc;
}

// block-wide argmax with the reference's scan semantics: the largest value, the lowest index among equals;
// idx < 0 = no candidate
__device__ void block_argmax(double& val, int& idx, double* s_val, int* s_idx) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 16; o > 0; o >>= 1) {
    const double ov = __shfl_down_sync(0xffffffffu, val, o);
    const int oi = __shfl_down_sync(0xffffffffu, idx, o);
    if (oi >= 0 && (idx < 0 || ov > val || (ov == val && oi < idx))) { val = ov; idx = oi; }
  }
  if (lane == 0) { s_val[warp] = val; s_idx[warp] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    double bv = s_val[0]; int bi = s_idx[0];
    for (int w = 1; w < DPP_THREADS / 32; ++w)
      if (s_idx[w] >= 0 && (bi < 0 || s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi))) { bv = s_val[w]; bi = s_idx[w]; }
    s_val[0] = bv; s_idx[0] = bi;
  }
  __syncthreads();
  val = s_val[0]; idx = s_idx[0];
  __syncthreads();
}

__global__ void __launch_bounds__(DPP_THREADS) dpp_rescore_kernel(DppKernelArgs a) {
  extern __shared__ __align__(16) unsigned char dsm[];
  const int b = blockIdx.x;
  const phx_dpp_config& cfg = a.cfg;
  const int C = a.in.num_candidates, E = a.in.emb_dim, Hc = a.in.num_context;
  const int n = a.in.num_valid ? min(max(a.in.num_valid[b], 0), C) : C;
  const int top_k = cfg.top_k;
  int* out_index = a.out_index + (size_t)b * top_k;
  double* out_score = a.out_score + (size_t)b * top_k;
  for (int i = threadIdx.x; i < top_k; i += DPP_THREADS) { out_index[i] = -1; out_score[i] = 0.0; }
  if (n == 0 || top_k == 0) { if (threadIdx.x == 0) a.out_count[b] = 0; return; }

  const double* score = a.in.scores + (size_t)b * C;
  const double* norm = a.in.norms + (size_t)b * C;
  const __half* emb = reinterpret_cast<const __half*>(a.in.embeddings) + (size_t)b * C * E;
  const uint8_t* missing = a.in.missing ? a.in.missing + (size_t)b * C : nullptr;
  const int* l1 = a.in.l1 ? a.in.l1 + (size_t)b * C : nullptr;
  const int n_ctx = Hc > 0 ? (a.in.num_context_valid ? min(max(a.in.num_context_valid[b], 0), Hc) : Hc) : 0;
  const __half* cemb = Hc > 0 ? reinterpret_cast<const __half*>(a.in.ctx_embeddings) + (size_t)b * Hc * E : nullptr;
  const double* cnorm = Hc > 0 ? a.in.ctx_norms + (size_t)b * Hc : nullptr;
  const uint8_t* cmissing = (Hc > 0 && a.in.ctx_missing) ? a.in.ctx_missing + (size_t)b * Hc : nullptr;
  const int* cl1 = (Hc > 0 && a.in.ctx_l1) ? a.in.ctx_l1 + (size_t)b * Hc : nullptr;

  const int m = min(cfg.max_selected_rank, n);
  const bool seed = !cfg.window_on && a.in.has_seed && n_ctx > 0;
  const int total = m + (seed ? 1 : 0);
  // shared: two [97 x 97] f64 matrices, then small per-item arrays
  double* K = reinterpret_cast<double*>(dsm);                       // kernel (or pool x pool cosines)
  double* Lc = K + (PHX_DPP_MAX_POOL + 1) * (PHX_DPP_MAX_POOL + 1);  // Cholesky rows (or context x pool cosines)
  double* qf = Lc + (PHX_DPP_MAX_POOL + 1) * (PHX_DPP_MAX_POOL + 1); // [97]
  double* wts = qf + (PHX_DPP_MAX_POOL + 1);                         // [128] window weights
  int* pool = reinterpret_cast<int*>(wts + 128);                     // [97] candidate index of pool position
  int* picked = pool + (PHX_DPP_MAX_POOL + 1);                       // [97] pick order (pool positions)
  int* avail = picked + (PHX_DPP_MAX_POOL + 1);                      // [97]
  int* recent = avail + (PHX_DPP_MAX_POOL + 1);                      // [128] window: most recent first; >= 0 pool position, < 0 context ~index
  __shared__ double s_val[DPP_THREADS / 32];
  __shared__ int s_idx[DPP_THREADS / 32];
  __shared__ int s_n;

  // ---- the pool: the m best scores, equal scores in input order ----
  for (int i = threadIdx.x; i < n; i += DPP_THREADS) {
    const double si = score[i];
    int rank = 0;
    for (int j = 0; j < n; ++j) { const double sj = score[j]; rank += (sj > si || (sj == si && j < i)) ? 1 : 0; }
    if (rank < m) pool[rank] = i;
  }
  __syncthreads();
  const double max_score = fmax(score[pool[0]], DPP_EPS);
  const double theta = fmin(fmax(cfg.theta, 0.0), 1.0 - DPP_EPS);
  const double alpha = theta / (2.0 * (1.0 - theta));
  int n_sel = 0;

  if (!cfg.window_on) {
    auto emb_at = [&](int ki) { return ki < m ? emb + (size_t)pool[ki] * E : cemb; };
    auto norm_at = [&](int ki) { return ki < m ? norm[pool[ki]] : cnorm[0]; };
    for (int ki = threadIdx.x; ki < total; ki += DPP_THREADS) {
      qf[ki] = exp(alpha * (ki < m ? score[pool[ki]] / max_score : 1.0));
      avail[ki] = 1;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < total * total; p += DPP_THREADS) {
      const int i = p / total, j = p % total;
      if (j < i) continue;
      double v;
      if (i == j) v = qf[i] * qf[i];
      else {
        const double denom = norm_at(i) * norm_at(j);
        const double cosv = denom > DPP_EPS ? dpp_dot(emb_at(i), emb_at(j), E) / denom : 0.0;
        v = qf[i] * qf[j] * cosv;
      }
      K[i * total + j] = v; K[j * total + i] = v;
    }
    __syncthreads();
    // greedy MAP (dpp.rs:282-369)
    const int pinned = (seed && K[m * total + m] > DPP_EPS) ? m : -1;
    const int max_items = pinned >= 0 ? min(top_k + 1, total) : min(top_k, total);
    double fv = -INFINITY; int fi = -1;
    if (pinned >= 0) { fv = K[pinned * total + pinned]; fi = pinned; }
    else {
      for (int i = threadIdx.x; i < total; i += DPP_THREADS) { const double d = K[i * total + i]; if (fi < 0 || d > fv) { fv = d; fi = i; } }
      block_argmax(fv, fi, s_val, s_idx);
    }
    if (threadIdx.x == 0) { picked[0] = fi; avail[fi] = 0; }
    {
      const double sq = sqrt(fv);
      for (int j = threadIdx.x; j < total; j += DPP_THREADS) Lc[j] = sq > DPP_EPS ? K[fi * total + j] / sq : 0.0;
    }
    __syncthreads();
    int count = 1;
    for (int s = 1; s < max_items; ++s) {
      double bv = -INFINITY; int bi = -1;
      for (int i = threadIdx.x; i < total; i += DPP_THREADS) {
        if (!avail[i]) continue;
        double cv = K[i * total + i];
        for (int j = 0; j < s; ++j) { const double f = Lc[j * total + i]; cv -= f * f; }
        if (bi < 0 || cv > bv) { bv = cv; bi = i; }
      }
      block_argmax(bv, bi, s_val, s_idx);
      if (bi < 0 || bv <= DPP_EPS) break;
      if (threadIdx.x == 0) { picked[s] = bi; avail[bi] = 0; }
      const double sq = sqrt(bv);
      for (int i = threadIdx.x; i < total; i += DPP_THREADS) {
        double sum = K[bi * total + i];
        for (int j = 0; j < s; ++j) sum -= Lc[j * total + bi] * Lc[j * total + i];
        Lc[s * total + i] = sum / sq;
      }
      __syncthreads();
      count = s + 1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {   // drop the seed from the picks
      int w = 0;
      for (int s = 0; s < count; ++s) if (picked[s] < m) picked[w++] = picked[s];
      s_n = w;
    }
    __syncthreads();
    n_sel = s_n;
  } else {
    // ---- sliding window (dpp.rs:371-413) ----
    auto cosine = [&](const __half* ea, double na, bool ma, const __half* eb, double nb, bool mb) {
      const double denom = na * nb;
      if (ma || mb || denom <= DPP_EPS) return 0.0;
      return dpp_dot(ea, eb, E) / denom;
    };
    for (int i = threadIdx.x; i < m; i += DPP_THREADS) {
      qf[i] = exp(2.0 * alpha * score[pool[i]] / max_score);
      avail[i] = 1;
    }
    for (int p = threadIdx.x; p < m * m; p += DPP_THREADS) {
      const int i = p / m, j = p % m;
      if (j < i) continue;
      const int ci = pool[i], cj = pool[j];
      const double v = cosine(emb + (size_t)ci * E, norm[ci], missing && missing[ci], emb + (size_t)cj * E, norm[cj], missing && missing[cj]);
      K[i * m + j] = v; K[j * m + i] = v;
    }
    long long size_ll = (long long)n_ctx + top_k;
    if ((long long)cfg.window_size < size_ll) size_ll = cfg.window_size;
    const int size = (int)(size_ll < 0 ? 0 : (size_ll > 128 ? 128 : size_ll));
    const int ctx_used = min(n_ctx, size);
    for (int p = threadIdx.x; p < ctx_used * m; p += DPP_THREADS) {
      const int c = p / m, j = p % m;
      const int cj = pool[j];
      Lc[c * m + j] = cosine(cemb + (size_t)c * E, cnorm[c], cmissing && cmissing[c], emb + (size_t)cj * E, norm[cj], missing && missing[cj]);
    }
    for (int d = threadIdx.x; d < size; d += DPP_THREADS)
      wts[d] = cfg.half_distance > 0.0 ? fmin(pow(0.5, (double)d / cfg.half_distance), 1.0) : 1.0;
    // most recent first: the context in its own order (item 0 is the most recent), picks are put in front as they come
    for (int d = threadIdx.x; d < 128; d += DPP_THREADS) recent[d] = (d < ctx_used) ? ~d : 0;
    __syncthreads();
    int n_recent = ctx_used;
    const int want = min(top_k, m);
    for (int step = 0; step < want; ++step) {
      double bv = -INFINITY; int bi = -1;
      for (int i = threadIdx.x; i < m; i += DPP_THREADS) {
        if (!avail[i]) continue;
        double g = qf[i];
        const int li = l1 ? l1[pool[i]] : -1;
        for (int d = 0; d < n_recent; ++d) {
          const int r = recent[d];
          double cs; int lr;
          if (r >= 0) { cs = K[r * m + i]; lr = l1 ? l1[pool[r]] : -1; }
          else { cs = Lc[(~r) * m + i]; lr = cl1 ? cl1[~r] : -1; }
          const double pen = fmin(cs * cs + ((lr >= 0 && lr == li) ? cfg.sid_lambda : 0.0), 1.0);
          g = g * (1.0 - wts[d] * pen);
        }
        if (bi < 0 || g > bv) { bv = g; bi = i; }
      }
      block_argmax(bv, bi, s_val, s_idx);
      if (bi < 0) break;
      if (threadIdx.x == 0) {
        avail[bi] = 0; picked[step] = bi;
        const int keep = min(n_recent, size - 1);          // the window holds `size` items: the new pick and the newest others
        for (int d = keep; d > 0; --d) recent[d] = recent[d - 1];
        if (size > 0) recent[0] = bi;
      }
      n_recent = size > 0 ? min(n_recent + 1, size) : 0;
      n_sel = step + 1;
      __syncthreads();
    }
  }

  // ---- serve (dpp.rs:192-215): positions in score order or pick order, scores always in score order ----
  if (threadIdx.x == 0) {
    int* by_score = avail;                     // reuse
    for (int s = 0; s < n_sel; ++s) by_score[s] = pool[picked[s]];
    for (int s = 1; s < n_sel; ++s) {          // insertion sort by (score desc, index asc); n_sel <= 96
      const int v = by_score[s]; const double sv = score[v];
      int t = s - 1;
      while (t >= 0 && (score[by_score[t]] < sv || (score[by_score[t]] == sv && by_score[t] > v))) { by_score[t + 1] = by_score[t]; --t; }
      by_score[t + 1] = v;
    }
    const bool pick_order = cfg.greedy_order || cfg.window_on;
    for (int s = 0; s < n_sel; ++s) {
      out_index[s] = pick_order ? pool[picked[s]] : by_score[s];
      out_score[s] = score[by_score[s]];
    }
    a.out_count[b] = n_sel;
  }
}

}  // namespace
}  // namespace phx

using namespace phx;

extern "C" phx_status phx_dpp_rescore_device(int32_t device, const phx_dpp_config* cfg, const phx_dpp_inputs* in, int32_t* out_index,
                                             double* out_score, int32_t* out_count, void* stream) {
  auto bad = [](const char* m) { set_global_error(std::string("phx_dpp_rescore_device: ") + m); return PHX_E_ARG; };
  if (!cfg || !in || !out_index || !out_score || !out_count) return bad("null argument");
  if (in->batch < 0 || in->num_candidates <= 0 || in->emb_dim <= 0 || in->num_context < 0) return bad("sizes");
  if (!in->scores || !in->embeddings || !in->norms) return bad("scores, embeddings and norms are required");
  if (cfg->top_k < 0 || cfg->top_k > PHX_DPP_MAX_POOL || cfg->max_selected_rank < 1 || cfg->max_selected_rank > PHX_DPP_MAX_POOL)
    return bad("top_k and max_selected_rank must be at most 96");
  if (in->num_context > PHX_DPP_MAX_CONTEXT) return bad("at most 32 context items (seed + history)");
  if (in->num_context > 0 && (!in->ctx_embeddings || !in->ctx_norms)) return bad("context embeddings and norms are required");
  if (cfg->window_on && cfg->window_size < 0) return bad("window size");
  if (in->batch == 0) return PHX_OK;
  if (cudaSetDevice(device) != cudaSuccess) { set_global_error("phx_dpp_rescore_device: cudaSetDevice failed"); return PHX_E_CUDA; }
  constexpr int N1 = PHX_DPP_MAX_POOL + 1;
  const size_t smem = (size_t)(2 * N1 * N1 + N1 + 128) * sizeof(double) + (size_t)(3 * N1 + 128) * sizeof(int);
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(dpp_rescore_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      set_global_error("phx_dpp_rescore_device: shared memory attribute"); return PHX_E_CUDA;
    }
    attr_set = true;
  }
  DppKernelArgs a;
  a.cfg = *cfg; a.in = *in; a.out_index = out_index; a.out_score = out_score; a.out_count = out_count;
  dpp_rescore_kernel<<<in->batch, DPP_THREADS, smem, (cudaStream_t)stream>>>(a);
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) { set_global_error(std::string("phx_dpp_rescore_device: ") + cudaGetErrorString(ce)); return PHX_E_CUDA; }
  return PHX_OK;
}
