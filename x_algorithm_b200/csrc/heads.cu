// Final RMSNorm of the candidate rows, the action and continuous heads, the server's log-sigmoid
// and the value-model blend in one pass (phoenix/xrex/models/recsys_model.py:4792-4843, 3557-3560,
// 3756-3846, 712-733; phoenix/xrex/inference/model_runner.py:4474; xai-value-model/scoring.rs:67-73,
// 112-120, 282-291).  One warp per candidate row; the (V+NC) x D head matrix sits in shared memory.
// Also the user-tower pooling (recsys_two_tower_model.py:2187-2200).
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace phx {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int MAX_OUT = 32;  // V + NC

__global__ void __launch_bounds__(256) heads_kernel(HeadsArgs a) {
  extern __shared__ __align__(16) uint8_t hsm[];
  bf16* sw = reinterpret_cast<bf16*>(hsm);  // [(V+NC), D]
  const int NO = a.V + a.NC;
  for (int i = threadIdx.x * 8; i < NO * a.D; i += blockDim.x * 8)
    *reinterpret_cast<uint4*>(sw + i) = *reinterpret_cast<const uint4*>(a.unembed_t + i);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long nrows = a.out_index ? a.rows : (long long)a.B * a.C;
  for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < nrows;
       r += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int b = (int)(r / a.C), c = (int)(r % a.C);
    // packed rows: candidate rows back to back, each answering the output slot out_index[r]
    const bf16* xr = a.out_index ? a.x + r * a.D : a.x + ((long long)b * a.T + a.S + c) * a.D;
    const long long orow = a.out_index ? a.out_index[r] : r;
    float ss = 0.f;
    for (int k = lane * 8; k < a.D; k += 256) {
      uint4 u = *reinterpret_cast<const uint4*>(xr + k);
      float2 p0 = unpack_bf2(u.x), p1 = unpack_bf2(u.y), p2 = unpack_bf2(u.z), p3 = unpack_bf2(u.w);
      ss += p0.x * p0.x + p0.y * p0.y + p1.x * p1.x + p1.y * p1.y + p2.x * p2.x + p2.y * p2.y + p3.x * p3.x + p3.y * p3.y;
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)a.D + a.eps);
    float acc[MAX_OUT];
#pragma unroll
    for (int j = 0; j < MAX_OUT; ++j) acc[j] = 0.f;
    for (int k = lane * 8; k < a.D; k += 256) {
      uint4 u = *reinterpret_cast<const uint4*>(xr + k);
      float xv[8];
      float2 p0 = unpack_bf2(u.x), p1 = unpack_bf2(u.y), p2 = unpack_bf2(u.z), p3 = unpack_bf2(u.w);
      xv[0] = p0.x; xv[1] = p0.y; xv[2] = p1.x; xv[3] = p1.y; xv[4] = p2.x; xv[5] = p2.y; xv[6] = p3.x; xv[7] = p3.y;
#pragma unroll
      for (int i = 0; i < 8; ++i) xv[i] = round_bf(xv[i] * rstd * a.final_gain[k + i]);  // normed row is bf16
#pragma unroll
      for (int j = 0; j < MAX_OUT; ++j) {
        if (j < NO) {
          uint4 w = *reinterpret_cast<const uint4*>(sw + j * a.D + k);
          float2 w0 = unpack_bf2(w.x), w1 = unpack_bf2(w.y), w2 = unpack_bf2(w.z), w3 = unpack_bf2(w.w);
          acc[j] += xv[0] * w0.x + xv[1] * w0.y + xv[2] * w1.x + xv[3] * w1.y + xv[4] * w2.x + xv[5] * w2.y + xv[6] * w3.x + xv[7] * w3.y;
        }
      }
    }
    // butterfly: 31 shuffles leave the total of output j on lane j (instead of 5 shuffles per output)
#pragma unroll
    for (int step = 16; step >= 1; step >>= 1) {
      const bool upper = (lane & step) != 0;
#pragma unroll
      for (int i = 0; i < step; ++i) {
        const float send = upper ? acc[i] : acc[i + step];
        const float keep = upper ? acc[i + step] : acc[i];
        acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, step);
      }
    }
    const float mine = acc[0];
    float value = 0.f;  // probability (f32 log-prob kept separately) or continuous prediction
    float logp = 0.f;
    if (lane < a.V) {
      float lg = round_bf(round_bf(mine) * a.output_scale);
      if (a.final_logit_cap > 0.f) lg = round_bf(a.final_logit_cap * tanhf(lg / a.final_logit_cap));
      logp = fminf(lg, 0.f) - log1pf(expf(-fabsf(lg)));  // log_sigmoid in fp32
      if (a.log_probs) a.log_probs[orow * a.V + lane] = logp;
    } else if (lane < NO) {
      float cl = round_bf(mine);
      float sg = round_bf(1.0f / (1.0f + expf(-cl)));
      value = round_bf(sg * a.dwell_norm_scale);
      if (a.continuous) a.continuous[orow * a.NC + (lane - a.V)] = value;
    }
    if (a.has_blend && a.scores) {
      // exp(ln p as f32 -> f64) like the client side; terms summed left to right in f64 by lane 0
      double col = (lane < a.V) ? exp((double)logp) : (double)value;
      double s = 0.0;
      for (int i = 0; i < a.blend.num_terms; ++i) {
        const int src = a.blend.src[i];
        double cv = __shfl_sync(0xffffffffu, col, src);
        s = s + cv * a.blend.weight[i];
      }
      if (lane == 0) {
        double out;
        if (a.blend.total_sum == 0.0) out = s > 0.0 ? s : 0.0;
        else if (s < 0.0) out = (s + a.blend.negative_sum) / a.blend.total_sum * 0.001;
        else out = s + 0.001;
        a.scores[orow] = out;
      }
    }
  }
}


// ---- tensor-core variant (D a multiple of 32) -----------------------------------------------------------------------
// One warp = 16 candidate rows.  The head matrix product runs on mma.sync m16n8k16: within every group of 32 columns
// the k index is permuted so that a thread's A fragments for two k-steps are one 16-byte load of its row (columns
// 8*t4 .. 8*t4+7 of the group) and its B fragments one 16-byte read of the head matrix row in shared memory.  Rows are
// normalised exactly like the scalar kernel (x * rstd * gain rounded to bf16) on their way into the fragments; the
// sums of squares come from a first pass over the same rows.  The per-output transcendental work is spread over all
// lanes ((row, output) items), the f64 blend runs one row per lane in the spec's term order.
constexpr int HM_WARPS = 8;
constexpr int HM_WPAD = 32;   // elements of padding per head-matrix row: rows g and g+1 fall into different bank halves

__device__ __forceinline__ void mma_bf16_16816_h(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NT>   // n-tiles of 8 outputs: V + NC <= 8 * NT
__global__ void __launch_bounds__(HM_WARPS * 32) heads_mma_kernel(HeadsArgs a) {
  extern __shared__ __align__(16) uint8_t hsm[];
  const int D = a.D, NO = a.V + a.NC, WLD = D + HM_WPAD;
  bf16* sw = reinterpret_cast<bf16*>(hsm);                                   // [NT*8][WLD], rows >= NO are zero
  float* sgain = reinterpret_cast<float*>(sw + NT * 8 * WLD);                // [D]
  float* sC_all = sgain + D;                                                 // per warp [16][NT*8] fp32 sums
  double* sD_all = reinterpret_cast<double*>(sC_all + HM_WARPS * 16 * NT * 8);   // per warp [16][NT*8] blend inputs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  for (int i = threadIdx.x; i < NT * 8 * (D / 8); i += blockDim.x) {
    const int n = i / (D / 8), ch = i % (D / 8);
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (n < NO) w = *reinterpret_cast<const uint4*>(a.unembed_t + (long long)n * D + ch * 8);
    *reinterpret_cast<uint4*>(sw + n * WLD + ch * 8) = w;
  }
  for (int i = threadIdx.x; i < D; i += blockDim.x) sgain[i] = a.final_gain[i];
  // programmatic dependent launch: the parameters above are staged while the last GEMM of the trunk drains; its
  // output is read only from here on
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();
  float* sC = sC_all + warp * 16 * NT * 8;
  double* sD = sD_all + warp * 16 * NT * 8;
  const long long nrows = a.out_index ? a.rows : (long long)a.B * a.C;
  const long long n_strips = (nrows + 15) / 16;
  const int groups = D / 32;
  for (long long strip = (long long)blockIdx.x * HM_WARPS + warp; strip < n_strips; strip += (long long)gridDim.x * HM_WARPS) {
    const long long r0 = strip * 16;
    const bf16* xr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      long long r = r0 + g + 8 * i;
      if (r >= nrows) r = nrows - 1;
      xr[i] = (a.out_index ? a.x + r * (long long)D : a.x + ((r / a.C) * a.T + a.S + (r % a.C)) * (long long)D) + 8 * t4;
    }
    // pass 1: sums of squares (a row's 32-column groups are spread over the 4 lanes of its quad)
    float ss[2] = {0.f, 0.f};
    for (int gr = 0; gr < groups; ++gr) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr[i] + gr * 32);
        const float2 p0 = unpack_bf2(u.x), p1 = unpack_bf2(u.y), p2 = unpack_bf2(u.z), p3 = unpack_bf2(u.w);
        ss[i] += (p0.x * p0.x + p0.y * p0.y) + (p1.x * p1.x + p1.y * p1.y) + (p2.x * p2.x + p2.y * p2.y) + (p3.x * p3.x + p3.y * p3.y);
      }
    }
    float rstd[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], 1);
      ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], 2);
      rstd[i] = rsqrtf(ss[i] / (float)D + a.eps);
    }
    // pass 2: normalise into A fragments, multiply
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
    for (int gr = 0; gr < groups; ++gr) {
      const float4 ga = *reinterpret_cast<const float4*>(sgain + gr * 32 + 8 * t4);
      const float4 gb = *reinterpret_cast<const float4*>(sgain + gr * 32 + 8 * t4 + 4);
      uint32_t fr[2][4];   // per row: the four packed pairs of its 8 normalised columns
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr[i] + gr * 32);
        const float2 p0 = unpack_bf2(u.x), p1 = unpack_bf2(u.y), p2 = unpack_bf2(u.z), p3 = unpack_bf2(u.w);
        fr[i][0] = pack_bf2(p0.x * rstd[i] * ga.x, p0.y * rstd[i] * ga.y);   // the normed row is bf16
        fr[i][1] = pack_bf2(p1.x * rstd[i] * ga.z, p1.y * rstd[i] * ga.w);
        fr[i][2] = pack_bf2(p2.x * rstd[i] * gb.x, p2.y * rstd[i] * gb.y);
        fr[i][3] = pack_bf2(p3.x * rstd[i] * gb.z, p3.y * rstd[i] * gb.w);
      }
      // k-step 0 uses pairs 0, 1 of each row, k-step 1 pairs 2, 3: fragment order [g][lo], [g+8][lo], [g][hi], [g+8][hi]
      const uint32_t a0[4] = {fr[0][0], fr[1][0], fr[0][1], fr[1][1]};
      const uint32_t a1[4] = {fr[0][2], fr[1][2], fr[0][3], fr[1][3]};
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint4 w = *reinterpret_cast<const uint4*>(sw + (j * 8 + g) * WLD + gr * 32 + 8 * t4);
        mma_bf16_16816_h(acc[j], a0, w.x, w.y);
        mma_bf16_16816_h(acc[j], a1, w.z, w.w);
      }
    }
    // the strip's 16 x (8 NT) sums to shared memory
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      *reinterpret_cast<float2*>(sC + g * (NT * 8) + j * 8 + 2 * t4) = make_float2(acc[j][0], acc[j][1]);
      *reinterpret_cast<float2*>(sC + (g + 8) * (NT * 8) + j * 8 + 2 * t4) = make_float2(acc[j][2], acc[j][3]);
    }
    __syncwarp();
    for (int idx = lane; idx < 16 * NO; idx += 32) {
      const int rr = idx / NO, oo = idx % NO;
      const long long r = r0 + rr;
      const long long orow = (a.out_index && r < nrows) ? a.out_index[r] : r;   // packed rows: the output slot this row answers
      const float mine = sC[rr * (NT * 8) + oo];
      double col;
      if (oo < a.V) {
        float lg = round_bf(round_bf(mine) * a.output_scale);
        if (a.final_logit_cap > 0.f) lg = round_bf(a.final_logit_cap * tanhf(lg / a.final_logit_cap));
        const float logp = fminf(lg, 0.f) - log1pf(expf(-fabsf(lg)));  // log_sigmoid in fp32
        if (a.log_probs && r < nrows) a.log_probs[orow * a.V + oo] = logp;
        col = a.has_blend ? exp((double)logp) : 0.0;   // exp(ln p as f32 -> f64) like the client side
      } else {
        const float cl = round_bf(mine);
        const float sg = round_bf(1.0f / (1.0f + expf(-cl)));
        const float value = round_bf(sg * a.dwell_norm_scale);
        if (a.continuous && r < nrows) a.continuous[orow * a.NC + (oo - a.V)] = value;
        col = (double)value;
      }
      sD[rr * (NT * 8) + oo] = col;
    }
    __syncwarp();
    if (a.has_blend && a.scores && lane < 16 && r0 + lane < nrows) {
      double s = 0.0;   // terms summed left to right in f64
      for (int i = 0; i < a.blend.num_terms; ++i) s = s + sD[lane * (NT * 8) + a.blend.src[i]] * a.blend.weight[i];
      double out;
      if (a.blend.total_sum == 0.0) out = s > 0.0 ? s : 0.0;
      else if (s < 0.0) out = (s + a.blend.negative_sum) / a.blend.total_sum * 0.001;
      else out = s + 0.001;
      a.scores[a.out_index ? a.out_index[r0 + lane] : r0 + lane] = out;
    }
    __syncwarp();
  }
}

template <int NT>
phx_status launch_heads_mma(const HeadsArgs& a, long long rows, cudaStream_t stream, std::string& err) {
  const size_t smem = (size_t)NT * 8 * (a.D + HM_WPAD) * sizeof(bf16) + (size_t)a.D * sizeof(float) +
                      (size_t)HM_WARPS * 16 * NT * 8 * (sizeof(float) + sizeof(double));
  if (smem > 200 * 1024) { err = "heads: head matrix does not fit shared memory"; return PHX_E_CAPACITY; }
  static bool attr_set = false;
  if (!attr_set) {
    PHX_CUDA_TRY(cudaFuncSetAttribute(heads_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), err);
    attr_set = true;
  }
  long long blocks = ((rows + 15) / 16 + HM_WARPS - 1) / HM_WARPS;
  if (blocks > 148 * 3) blocks = 148 * 3;
  cudaLaunchConfig_t lc;
  memset(&lc, 0, sizeof(lc));
  lc.gridDim = dim3((unsigned)blocks); lc.blockDim = dim3(HM_WARPS * 32); lc.dynamicSmemBytes = smem; lc.stream = stream;
  cudaLaunchAttribute at[1];
  static const bool pdl = !(getenv("PHX_PDL") && getenv("PHX_PDL")[0] == '0');
  if (pdl) {   // start while the kernel in front drains; the kernel waits before it reads the residual stream
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
  }
  PHX_CUDA_TRY(cudaLaunchKernelEx(&lc, heads_mma_kernel<NT>, a), err);
  return PHX_OK;
}

// users[b] = l2norm(mean over valid t of final_norm(x[b,t])), fp32; one CTA per user, one thread per column
template <bool F32>   // F32: fp32 rows, nothing rounded (the full-precision path)
__global__ void tower_pool_kernel(const void* __restrict__ xv, const float* __restrict__ gain, const int* __restrict__ seg,
                                  int T, int D, float eps, float* __restrict__ users) {
  auto ld = [&](long long i) { return F32 ? reinterpret_cast<const float*>(xv)[i] : bf2f(reinterpret_cast<const bf16*>(xv)[i]); };
  extern __shared__ float psm[];  // [T] rstd (0 for invalid) + reduction scratch
  float* rstd = psm;
  float* red = psm + T;
  const int b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int t = warp; t < T; t += nw) {
    const long long r0 = ((long long)b * T + t) * D;
    float ss = 0.f;
    for (int k = lane; k < D; k += 32) { float v = ld(r0 + k); ss += v * v; }
    ss = warp_sum(ss);
    if (lane == 0) rstd[t] = (seg[(long long)b * T + t] != 0) ? (F32 ? 1.0f / sqrtf(ss / (float)D + eps) : rsqrtf(ss / (float)D + eps)) : 0.f;
  }
  __syncthreads();
  float cnt = 0.f;
  for (int t = 0; t < T; ++t) cnt += (rstd[t] != 0.f) ? 1.f : 0.f;
  float sq = 0.f;
  float vals[8];  // D <= 8 * blockDim.x
  int nv = 0;
  for (int k = threadIdx.x; k < D; k += blockDim.x, ++nv) {
    float acc = 0.f;
    const float gk = gain[k];
    for (int t = 0; t < T; ++t) {  // fixed order over positions
      if (rstd[t] != 0.f) {
        const float v = ld(((long long)b * T + t) * D + k) * rstd[t] * gk;
        acc = acc + (F32 ? v : round_bf(v));
      }
    }
    const float rep = acc / fmaxf(cnt, 1.0f);
    vals[nv] = rep;
    sq += rep * rep;
  }
  sq = warp_sum(sq);
  if (lane == 0) red[warp] = sq;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < nw; ++w) tot += red[w];
  const float inv = 1.0f / sqrtf(fmaxf(tot, 1e-12f));
  nv = 0;
  for (int k = threadIdx.x; k < D; k += blockDim.x, ++nv) users[(long long)b * D + k] = vals[nv] * inv;
}

}  // namespace

phx_status heads_launch(const HeadsArgs& a, cudaStream_t stream, std::string& err) {
  const int NO = a.V + a.NC;
  if (NO > MAX_OUT || a.D % 8 != 0) { err = "heads: V + NC must be <= 32 and D a multiple of 8"; return PHX_E_ARG; }
  if (a.has_blend) {
    for (int i = 0; i < a.blend.num_terms; ++i)
      if (a.blend.src[i] < 0 || a.blend.src[i] >= NO) { err = "heads: blend term source out of range"; return PHX_E_ARG; }
  }
  const long long rows = a.out_index ? a.rows : (long long)a.B * a.C;
  if (rows == 0) return PHX_OK;
  if (a.D % 32 == 0 && !(getenv("PHX_HEADS") && strcmp(getenv("PHX_HEADS"), "scalar") == 0)) {   // tensor-core path
    if (NO <= 8) return launch_heads_mma<1>(a, rows, stream, err);
    if (NO <= 16) return launch_heads_mma<2>(a, rows, stream, err);
    if (NO <= 24) return launch_heads_mma<3>(a, rows, stream, err);
    return launch_heads_mma<4>(a, rows, stream, err);
  }
  const size_t smem = (size_t)NO * a.D * sizeof(bf16);
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    PHX_CUDA_TRY(cudaFuncSetAttribute(heads_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), err);
    attr_set = true;
  }
  if (smem > 200 * 1024) { err = "heads: head matrix does not fit shared memory"; return PHX_E_CAPACITY; }
  long long blocks = (rows + 7) / 8;
  if (blocks > 148 * 4) blocks = 148 * 4;
  heads_kernel<<<(unsigned)blocks, 256, smem, stream>>>(a);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status tower_pool_launch(const void* x, const float* final_gain, const int* seg, int B, int T, int D, float eps,
                             float* users, cudaStream_t stream, std::string& err, bool x_is_f32) {
  if (B == 0) return PHX_OK;
  int threads = 256;
  if (D > 8 * threads) { err = "tower_pool: D too large"; return PHX_E_CAPACITY; }
  const size_t smem = (size_t)(T + 32) * sizeof(float);
  if (x_is_f32) tower_pool_kernel<true><<<B, threads, smem, stream>>>(x, final_gain, seg, T, D, eps, users);
  else tower_pool_kernel<false><<<B, threads, smem, stream>>>(x, final_gain, seg, T, D, eps, users);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

}  // namespace phx
