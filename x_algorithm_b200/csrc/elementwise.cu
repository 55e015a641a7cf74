// RMSNorm (phoenix/xrex/models/normalization.py:110-122), joint all-heads qk-norm
// (normalization.py:46-48) and RoPE (phoenix/xrex/models/layers.py:52-67, 784-788) as
// HBM-bound row kernels: one warp per token row, 16-byte loads, fp32 math, bf16 stores.
#include "common.cuh"

namespace phx {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// y = bf16(norm(x)) or, with a residual, y = bf16(res + bf16(norm(x))); y may alias x or res
__global__ void __launch_bounds__(256) rmsnorm_kernel(const bf16* x, const float* __restrict__ gain, bf16* y,
                                                      const bf16* res, long long rows, int D, float eps) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + row * D;
  float ss = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    uint4 u = *reinterpret_cast<const uint4*>(xr + c);
    float2 a = unpack_bf2(u.x), b = unpack_bf2(u.y), cc = unpack_bf2(u.z), d = unpack_bf2(u.w);
    ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + cc.x * cc.x + cc.y * cc.y + d.x * d.x + d.y * d.y;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)D + eps);
  for (int c = lane * 8; c < D; c += 256) {
    uint4 u = *reinterpret_cast<const uint4*>(xr + c);
    float4 g0 = *reinterpret_cast<const float4*>(gain + c);
    float4 g1 = *reinterpret_cast<const float4*>(gain + c + 4);
    float2 a = unpack_bf2(u.x), b = unpack_bf2(u.y), cc = unpack_bf2(u.z), d = unpack_bf2(u.w);
    float v[8] = {a.x * rstd * g0.x, a.y * rstd * g0.y, b.x * rstd * g0.z, b.y * rstd * g0.w,
                  cc.x * rstd * g1.x, cc.y * rstd * g1.y, d.x * rstd * g1.z, d.y * rstd * g1.w};
    if (res) {
      uint4 ru = *reinterpret_cast<const uint4*>(res + row * D + c);
      float2 r0 = unpack_bf2(ru.x), r1 = unpack_bf2(ru.y), r2 = unpack_bf2(ru.z), r3 = unpack_bf2(ru.w);
      const float rv[8] = {r0.x, r0.y, r1.x, r1.y, r2.x, r2.y, r3.x, r3.y};
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = round_bf(v[i]) + rv[i];
    }
    uint4 o;
    o.x = pack_bf2(v[0], v[1]); o.y = pack_bf2(v[2], v[3]); o.z = pack_bf2(v[4], v[5]); o.w = pack_bf2(v[6], v[7]);
    *reinterpret_cast<uint4*>(y + row * D + c) = o;
  }
}

// In place on the merged qkv row of one token.  Column of element d of q head h:
// ((h / g) * (g + 2) + h % g) * dh + d; of k head j: (j * (g + 2) + g) * dh + d  (layers.py:728-736).
__global__ void __launch_bounds__(256) qknorm_rope_kernel(QkNormRopeArgs a) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= a.M) return;
  const int g = a.Hq / a.Hkv, dh = a.dh, half = dh >> 1;
  const int width = (a.Hq + 2 * a.Hkv) * dh;
  bf16* r = a.qkv + row * width;
  int pos = a.pos_cap;   // split layout (GemmRope): the candidate block sits at the cap
  if (a.pos_rows) {
    pos = a.pos_rows[row + a.row_offset];
  } else if (a.split_rows == 0 || row + a.row_offset < a.split_rows) {
    const int t = (int)((row + a.row_offset) % a.T);
    pos = t < a.pos_cap ? t : a.pos_cap;
  }
  const float* ct = a.cos_tab + (long long)pos * half;
  const float* st = a.sin_tab + (long long)pos * half;
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {  // 0 = q heads, 1 = k heads
    const int nheads = which == 0 ? a.Hq : a.Hkv;
    const float* gain = which == 0 ? a.q_gain : a.k_gain;
    float rstd = 1.f;
    if (a.qk_norm) {
      float ss = 0.f;
      for (int e = lane; e < nheads * dh; e += 32) {
        const int h = e / dh, d = e % dh;
        const int col = (which == 0 ? ((h / g) * (g + 2) + h % g) : (h * (g + 2) + g)) * dh + d;
        const float v = bf2f(r[col]);
        ss += v * v;
      }
      ss = warp_sum(ss);
      rstd = rsqrtf(ss / (float)(nheads * dh) + 1e-5f);
    }
    for (int e = lane; e < nheads * half; e += 32) {
      const int h = e / half, j = e % half;
      const int base = (which == 0 ? ((h / g) * (g + 2) + h % g) : (h * (g + 2) + g)) * dh;
      float x1 = bf2f(r[base + j]), x2 = bf2f(r[base + j + half]);
      if (a.qk_norm) {  // normed values are materialised in bf16 before RoPE
        x1 = round_bf(x1 * rstd * gain[h * dh + j]);
        x2 = round_bf(x2 * rstd * gain[h * dh + j + half]);
      }
      if (a.rotary) {
        const float c = ct[j], s = st[j];
        const float y1 = x1 * c - x2 * s;  // x*cos + rotate_half(x)*sin, rotate_half = (-x2, x1)
        const float y2 = x2 * c + x1 * s;
        x1 = y1; x2 = y2;
      }
      r[base + j] = f2bf(x1);
      r[base + j + half] = f2bf(x2);
    }
  }
}

// out[n][k] = bf16(w_t[n][k] * gain[k]): a norm's gain folded into the K-major weight of the GEMM that follows it
__global__ void fold_gain_kernel(const bf16* __restrict__ w_t, const float* __restrict__ gain, bf16* __restrict__ out,
                                 long long total, int K) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    out[i] = f2bf(bf2f(w_t[i]) * gain[i % K]);
}

}  // namespace

phx_status fold_gain_launch(const bf16* w_t, const float* gain, bf16* out, int N, int K, cudaStream_t stream,
                            std::string& err) {
  const long long total = (long long)N * K;
  fold_gain_kernel<<<(unsigned)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256), 256, 0, stream>>>(w_t, gain, out, total, K);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status rmsnorm_launch(const bf16* x, const float* gain, bf16* y, const bf16* res, long long rows, int D, float eps,
                          cudaStream_t stream, std::string& err) {
  if (D % 8 != 0) { err = "rmsnorm: D must be a multiple of 8"; return PHX_E_ARG; }
  if (rows == 0) return PHX_OK;
  rmsnorm_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(x, gain, y, res, rows, D, eps);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status qknorm_rope_launch(const QkNormRopeArgs& a, cudaStream_t stream, std::string& err) {
  if (a.M == 0 || (!a.rotary && !a.qk_norm)) return PHX_OK;
  qknorm_rope_kernel<<<(unsigned)((a.M + 7) / 8), 256, 0, stream>>>(a);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

}  // namespace phx
