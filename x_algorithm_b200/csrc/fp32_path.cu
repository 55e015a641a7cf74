// Full-precision ranking forward: every activation in fp32, weights the same bf16-representable values as the bf16
// path (stored bf16, so the products are exact fp32 products of the reference's fp32 parameters).  This is the
// precision path of the reference's CPU-runnable configuration (fp32 model, phoenix/xrex/models/transformer.py:461-618,
// layers.py:52-67, 340-371, normalization.py:46-48, 110-122, pallas/ranker_attention_v2.py:113-148, 183), kept as
// plain SIMT kernels: it exists to pin the engine's arithmetic against the fp32 model to ~1e-6, not for throughput
// (the bf16 tcgen05 kernels are the throughput path).  Token rows are in plain [B, T] order.
#include "common.cuh"

namespace phx {
namespace {

__device__ __forceinline__ float warp_sum32(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max32(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// jax.nn.gelu(approximate=True) with the library tanhf (the bf16 path's tanh.approx is too coarse here)
__device__ __forceinline__ float gelu_tanh_exact(float x) {
  const float c = 0.7978845608028654f;  // sqrt(2/pi)
  return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
}

// y = norm(x) * gain, or res + norm(x) * gain; one warp per row; y may alias x or res
__global__ void __launch_bounds__(256) f32_rmsnorm_kernel(const float* x, const float* __restrict__ gain, float* y,
                                                          const float* res, long long rows, int D, float eps) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float* xr = x + row * D;
  float ss = 0.f;
  for (int c = lane; c < D; c += 32) ss += xr[c] * xr[c];
  ss = warp_sum32(ss);
  const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
  for (int c = lane; c < D; c += 32) {
    const float v = rstd * xr[c] * gain[c];
    y[row * D + c] = res ? res[row * D + c] + v : v;
  }
}

// C[M,N] = epi(A[M,K] @ Wt[N,K]^T): 64 x 64 tile per CTA, 4 x 4 outputs per thread, k in steps of 16.
constexpr int FT = 64, FK = 16;
template <int EPI>
__global__ void __launch_bounds__(256) f32_gemm_kernel(const float* __restrict__ A, const bf16* __restrict__ Wt, float* C,
                                                       const float* R, long long M, int N, int K) {
  __shared__ float sa[FK][FT + 4];
  __shared__ float sb[FK][FT + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long m0 = (long long)blockIdx.y * FT;
  const int n0 = blockIdx.x * FT;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += FK) {
    for (int i = threadIdx.x; i < FT * FK; i += 256) {
      const int r = i / FK, kk = i % FK;
      const long long row = m0 + r;
      sa[kk][r] = (row < M && k0 + kk < K) ? A[row * K + k0 + kk] : 0.f;
      const int wr = n0 + r;
      sb[kk][r] = (wr < N && k0 + kk < K) ? bf2f(Wt[(long long)wr * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < FK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = sa[kk][ty * 4 + i]; bv[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long row = m0 + ty * 4 + i;
    if (row >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col >= N) continue;
      float v = acc[i][j];
      if (EPI == EPI_RESIDUAL) v += R[row * N + col];
      else if (EPI == EPI_GELU) v = gelu_tanh_exact(v);
      C[row * N + col] = v;
    }
  }
}

// joint all-heads qk-norm and RoPE in place on the merged fp32 qkv row of one token; one warp per row.
// Column of element d of q head h: ((h / g) * (g + 2) + h % g) * dh + d; of k head j: (j * (g + 2) + g) * dh + d.
__global__ void __launch_bounds__(256) f32_qknorm_rope_kernel(float* qkv, long long M, int T, int Hq, int Hkv, int dh,
                                                              int pos_cap, int rotary, int qk_norm, const float* q_gain,
                                                              const float* k_gain, const float* cos_tab, const float* sin_tab) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const int g = Hq / Hkv, half = dh >> 1;
  float* r = qkv + row * (long long)((Hq + 2 * Hkv) * dh);
  const int t = (int)(row % T);
  const int pos = t < pos_cap ? t : pos_cap;
  const float* ct = cos_tab + (long long)pos * half;
  const float* st = sin_tab + (long long)pos * half;
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {
    const int nheads = which == 0 ? Hq : Hkv;
    const float* gain = which == 0 ? q_gain : k_gain;
    float rstd = 1.f;
    if (qk_norm) {
      float ss = 0.f;
      for (int e = lane; e < nheads * dh; e += 32) {
        const int h = e / dh, d = e % dh;
        const float v = r[(which == 0 ? ((h / g) * (g + 2) + h % g) : (h * (g + 2) + g)) * dh + d];
        ss += v * v;
      }
      ss = warp_sum32(ss);
      rstd = 1.0f / sqrtf(ss / (float)(nheads * dh) + 1e-5f);
    }
    for (int e = lane; e < nheads * half; e += 32) {
      const int h = e / half, j = e % half;
      const int base = (which == 0 ? ((h / g) * (g + 2) + h % g) : (h * (g + 2) + g)) * dh;
      float x1 = r[base + j], x2 = r[base + j + half];
      if (qk_norm) { x1 = rstd * x1 * gain[h * dh + j]; x2 = rstd * x2 * gain[h * dh + j + half]; }
      if (rotary) {
        const float c = ct[j], s = st[j];
        const float y1 = x1 * c - x2 * s, y2 = x2 * c + x1 * s;
        x1 = y1; x2 = y2;
      }
      r[base + j] = x1; r[base + j + half] = x2;
    }
  }
}

// Candidate-isolation attention in fp32: one warp per (request, head, query row).  Allowed keys: every history key
// with segment id 1, plus the query's own position (ranker_attention_v2.py:131-132); a padded query row gives 0
// (line 183).  Two passes over the scores (maximum, then exp / sum / P V), so the softmax is the plain fp32 one.
__global__ void __launch_bounds__(256) f32_attention_kernel(const float* __restrict__ qkv, const int* __restrict__ seg,
                                                            float* __restrict__ out, int B, int T, int Hq, int Hkv, int dh,
                                                            int hist_len, float sm_scale, float cap, int cap_method) {
  extern __shared__ float fsm[];   // per warp: scores of the history keys + self [hist + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int n_hist = hist_len < T ? hist_len : T;
  float* sc = fsm + (size_t)warp * (n_hist + 1);
  const int g = Hq / Hkv;
  const int QW = (Hq + 2 * Hkv) * dh;
  const long long nq = (long long)B * Hq * T;
  for (long long item = (long long)blockIdx.x * nw + warp; item < nq; item += (long long)gridDim.x * nw) {
    const int t = (int)(item % T);
    const int h = (int)((item / T) % Hq);
    const int b = (int)(item / ((long long)T * Hq));
    const long long tok0 = (long long)b * T;
    float* o = out + ((tok0 + t) * Hq + h) * dh;
    const int sq = seg[tok0 + t];
    if (sq == 0) {
      for (int d = lane; d < dh; d += 32) o[d] = 0.f;
      continue;
    }
    const int hk = h / g;
    const float* q = qkv + (tok0 + t) * QW + ((h / g) * (g + 2) + h % g) * dh;
    const int koff = (hk * (g + 2) + g) * dh, voff = koff + dh;
    const bool self_extra = !(t < n_hist && sq == 1);   // a valid history query already has itself among the history keys
    const int nk = n_hist + (self_extra ? 1 : 0);
    // pass 1: scores (each lane whole dot products), running maximum
    float mx = -INFINITY;
    for (int k = lane; k < nk; k += 32) {
      const int kt = k < n_hist ? k : t;
      const bool ok = k >= n_hist || seg[tok0 + kt] == 1;
      float s = -INFINITY;
      if (ok) {
        const float* kr = qkv + (tok0 + kt) * QW + koff;
        float acc = 0.f;
        for (int d = 0; d < dh; ++d) acc = fmaf(q[d], kr[d], acc);
        s = acc * sm_scale;
        if (cap_method == 1) s = s / (1.0f + fabsf(s) / cap);
        else if (cap_method == 2) s = cap * tanhf(s / cap);
      }
      sc[k] = s;
      mx = fmaxf(mx, s);
    }
    mx = warp_max32(mx);
    __syncwarp();
    float l = 0.f;
    for (int k = lane; k < nk; k += 32) {
      const float p = sc[k] == -INFINITY ? 0.f : expf(sc[k] - mx);
      sc[k] = p;
      l += p;
    }
    l = warp_sum32(l);
    __syncwarp();
    // pass 2: O = P V, lanes over the head dim
    for (int d = lane; d < dh; d += 32) {
      float acc = 0.f;
      for (int k = 0; k < nk; ++k) {
        const float p = sc[k];
        if (p != 0.f) acc = fmaf(p, qkv[(tok0 + (k < n_hist ? k : t)) * QW + voff + d], acc);
      }
      o[d] = acc / (l == 0.f ? 1.0f : l);
    }
    __syncwarp();
  }
}

// Final RMSNorm of the candidate rows, heads, log-sigmoid and blend in fp32 (the f64 blend as in the bf16 path):
// one warp per candidate row, lane j ends up with output j.
__global__ void __launch_bounds__(256) f32_heads_kernel(const float* __restrict__ x, HeadsArgs a) {
  const int lane = threadIdx.x & 31;
  const int NO = a.V + a.NC;
  const long long nrows = (long long)a.B * a.C;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= nrows) return;
  const int b = (int)(r / a.C), c = (int)(r % a.C);
  const float* xr = x + ((long long)b * a.T + a.S + c) * a.D;
  float ss = 0.f;
  for (int k = lane; k < a.D; k += 32) ss += xr[k] * xr[k];
  ss = warp_sum32(ss);
  const float rstd = 1.0f / sqrtf(ss / (float)a.D + a.eps);
  float mine = 0.f;
  for (int j = 0; j < NO; ++j) {
    float acc = 0.f;
    for (int k = lane; k < a.D; k += 32) acc = fmaf(rstd * xr[k] * a.final_gain[k], bf2f(a.unembed_t[(long long)j * a.D + k]), acc);
    acc = warp_sum32(acc);
    if (lane == j) mine = acc;
  }
  float value = 0.f, logp = 0.f;
  if (lane < a.V) {
    float lg = mine * a.output_scale;
    if (a.final_logit_cap > 0.f) lg = a.final_logit_cap * tanhf(lg / a.final_logit_cap);
    logp = fminf(lg, 0.f) - log1pf(expf(-fabsf(lg)));
    if (a.log_probs) a.log_probs[r * a.V + lane] = logp;
  } else if (lane < NO) {
    value = (1.0f / (1.0f + expf(-mine))) * a.dwell_norm_scale;
    if (a.continuous) a.continuous[r * a.NC + (lane - a.V)] = value;
  }
  if (a.has_blend && a.scores) {
    double col = (lane < a.V) ? exp((double)logp) : (double)value;
    double s = 0.0;
    for (int i = 0; i < a.blend.num_terms; ++i) {
      const double cv = __shfl_sync(0xffffffffu, col, a.blend.src[i]);
      s = s + cv * a.blend.weight[i];
    }
    if (lane == 0) {
      double o;
      if (a.blend.total_sum == 0.0) o = s > 0.0 ? s : 0.0;
      else if (s < 0.0) o = (s + a.blend.negative_sum) / a.blend.total_sum * 0.001;
      else o = s + 0.001;
      a.scores[r] = o;
    }
  }
}

}  // namespace

phx_status f32_rmsnorm_launch(const float* x, const float* gain, float* y, const float* res, long long rows, int D, float eps,
                              cudaStream_t stream, std::string& err) {
  if (rows == 0) return PHX_OK;
  f32_rmsnorm_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(x, gain, y, res, rows, D, eps);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status f32_gemm_launch(const float* A, const bf16* Wt, float* C, const float* R, int64_t M, int N, int K, int epilogue,
                           cudaStream_t stream, std::string& err) {
  if (M == 0) return PHX_OK;
  const int64_t chunk = 65535LL * FT;   // gridDim.y limit
  for (int64_t m0 = 0; m0 < M; m0 += chunk) {
    const int64_t mm = (M - m0 < chunk) ? (M - m0) : chunk;
    dim3 grid((N + FT - 1) / FT, (unsigned)((mm + FT - 1) / FT));
    const float* a = A + m0 * K; float* c = C + m0 * N; const float* r = R ? R + m0 * N : nullptr;
    switch (epilogue) {
      case EPI_STORE: f32_gemm_kernel<EPI_STORE><<<grid, 256, 0, stream>>>(a, Wt, c, r, mm, N, K); break;
      case EPI_RESIDUAL:
        if (!R) { err = "fp32 gemm: residual epilogue needs R"; return PHX_E_ARG; }
        f32_gemm_kernel<EPI_RESIDUAL><<<grid, 256, 0, stream>>>(a, Wt, c, r, mm, N, K); break;
      case EPI_GELU: f32_gemm_kernel<EPI_GELU><<<grid, 256, 0, stream>>>(a, Wt, c, r, mm, N, K); break;
      default: err = "fp32 gemm: unknown epilogue"; return PHX_E_ARG;
    }
    PHX_CUDA_TRY(cudaGetLastError(), err);
  }
  return PHX_OK;
}

phx_status f32_qknorm_rope_launch(float* qkv, long long M, int T, int Hq, int Hkv, int dh, int pos_cap, int rotary, int qk_norm,
                                  const float* q_gain, const float* k_gain, const float* cos_tab, const float* sin_tab,
                                  cudaStream_t stream, std::string& err) {
  if (M == 0 || (!rotary && !qk_norm)) return PHX_OK;
  f32_qknorm_rope_kernel<<<(unsigned)((M + 7) / 8), 256, 0, stream>>>(qkv, M, T, Hq, Hkv, dh, pos_cap, rotary, qk_norm, q_gain,
                                                                      k_gain, cos_tab, sin_tab);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status f32_attention_launch(const float* qkv, const int* seg, float* out, int B, int T, int Hq, int Hkv, int dh,
                                int hist_len, float sm_scale, float cap, int cap_method, cudaStream_t stream, std::string& err) {
  if (B == 0 || T == 0) return PHX_OK;
  const int n_hist = hist_len < T ? hist_len : T;
  int warps = 8;
  while (warps > 1 && (size_t)warps * (n_hist + 1) * sizeof(float) > 200 * 1024) warps >>= 1;
  const size_t smem = (size_t)warps * (n_hist + 1) * sizeof(float);
  if (smem > 200 * 1024) { err = "fp32 attention: history too long for the score buffer"; return PHX_E_CAPACITY; }
  if (smem > 48 * 1024)
    PHX_CUDA_TRY(cudaFuncSetAttribute(f32_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), err);
  const long long items = (long long)B * Hq * T;
  long long blocks = (items + warps - 1) / warps;
  if (blocks > 148 * 64) blocks = 148 * 64;
  f32_attention_kernel<<<(unsigned)blocks, warps * 32, smem, stream>>>(qkv, seg, out, B, T, Hq, Hkv, dh, hist_len, sm_scale,
                                                                       cap, cap_method);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status f32_heads_launch(const float* x, const HeadsArgs& a, cudaStream_t stream, std::string& err) {
  const long long nrows = (long long)a.B * a.C;
  if (nrows == 0) return PHX_OK;
  if (a.V + a.NC > 32) { err = "heads: at most 32 outputs"; return PHX_E_ARG; }
  f32_heads_kernel<<<(unsigned)((nrows + 7) / 8), 256, 0, stream>>>(x, a);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

}  // namespace phx
