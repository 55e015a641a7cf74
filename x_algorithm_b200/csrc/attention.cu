// Candidate-isolated ("ranker") attention: every valid query attends to the valid history keys, a
// candidate additionally to itself and to no other candidate, padded queries produce zeros
// (mask: phoenix/xrex/pallas/ranker_attention_utils.py:16-56; kernel form
// phoenix/xrex/pallas/ranker_attention_v2.py:113-148, 183).
//
// The candidate x candidate block is never formed: the kernel streams only the history keys
// through shared memory (64 keys per step) and folds the candidate's single self key in as one
// extra online-softmax step computed as a per-row dot product.  One CTA = 64 query rows of one
// (batch, head): 4 warps x 16 rows, Q fragments in registers, S = Q K^T and O += P V on
// mma.sync m16n8k16 bf16 with fp32 accumulation, P rounded to bf16 before P V as the reference does.
#include "common.cuh"

namespace phx {
namespace {

constexpr int KB = 64;        // keys per step
constexpr int QROWS = 64;     // query rows per CTA
constexpr int ATT_THREADS = 128;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ float cap_logit(float s, float cap, int method) {
  if (method == 1) return s / (1.0f + fabsf(s) / cap);   // soft_sign
  if (method == 2) return cap * tanhf(s / cap);          // tanh
  return s;
}

template <int DH>
__global__ void __launch_bounds__(ATT_THREADS) ranker_attention_kernel(AttnArgs a) {
  constexpr int LD = DH + 8;          // padded row (elements): conflict-free fragment loads
  constexpr int KSTEPS = DH / 16;     // k-steps of Q K^T
  constexpr int DT = DH / 8;          // output n-tiles
  __shared__ __align__(16) bf16 sk[KB * LD];
  __shared__ __align__(16) bf16 sv[KB * LD];
  __shared__ int skey_ok[KB];

  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * QROWS;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int T = a.T;
  const float LOG2E = 1.4426950408889634f;

  // rows of this thread: r0 = q0 + warp*16 + g, r1 = r0 + 8
  const int rq[2] = {q0 + warp * 16 + g, q0 + warp * 16 + g + 8};
  int segq[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) segq[i] = (rq[i] < T) ? a.seg[(long long)b * T + rq[i]] : 0;

  // Q fragments straight from global memory
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const bf16* qp = a.q + ((long long)b * T + rq[i]) * a.q_tok_stride + (long long)h * a.q_head_stride + ks * 16 + 2 * t4;
      const bool ok = rq[i] < T;
      qf[ks][i] = ok ? *reinterpret_cast<const uint32_t*>(qp) : 0u;
      qf[ks][i + 2] = ok ? *reinterpret_cast<const uint32_t*>(qp + 8) : 0u;
    }
  }

  float o[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const int n_hist = a.hist_len < T ? a.hist_len : T;
  for (int k0 = 0; k0 < n_hist; k0 += KB) {
    __syncthreads();
    // stage K and V rows k0..k0+KB of this (batch, kv head): 16-byte chunks
    for (int c = threadIdx.x; c < KB * (DH / 8); c += ATT_THREADS) {
      const int kr = c / (DH / 8), dc = (c % (DH / 8)) * 8;
      const int key = k0 + kr;
      uint4 uk = make_uint4(0, 0, 0, 0), uv = make_uint4(0, 0, 0, 0);
      if (key < n_hist) {
        uk = *reinterpret_cast<const uint4*>(a.k + ((long long)b * T + key) * a.k_tok_stride + (long long)hk * a.k_head_stride + dc);
        uv = *reinterpret_cast<const uint4*>(a.v + ((long long)b * T + key) * a.v_tok_stride + (long long)hk * a.v_head_stride + dc);
      }
      *reinterpret_cast<uint4*>(&sk[kr * LD + dc]) = uk;
      *reinterpret_cast<uint4*>(&sv[kr * LD + dc]) = uv;
    }
    if (threadIdx.x < KB) {
      const int key = k0 + threadIdx.x;
      skey_ok[threadIdx.x] = (key < n_hist) && (a.seg[(long long)b * T + key] == 1);
    }
    __syncthreads();

    // S = Q K^T for 64 keys: 8 n-tiles of 8 keys
    float s[KB / 8][4];
#pragma unroll
    for (int j = 0; j < KB / 8; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const bf16* kp = &sk[(j * 8 + g) * LD + ks * 16 + 2 * t4];
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kp);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kp + 8);
        mma_bf16_16816(s[j], qf[ks], b0, b1);
      }
    }
    // scale, cap, mask, block max
    float bm[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < KB / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kc = j * 8 + 2 * t4 + (e & 1);
        const int ri = e >> 1;
        float v = cap_logit(s[j][e] * a.sm_scale, a.cap, a.cap_method);
        const bool ok = skey_ok[kc] && segq[ri] != 0;
        v = ok ? v : -INFINITY;
        s[j][e] = v;
        bm[ri] = fmaxf(bm[ri], v);
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      bm[i] = fmaxf(bm[i], __shfl_xor_sync(0xffffffffu, bm[i], 1));
      bm[i] = fmaxf(bm[i], __shfl_xor_sync(0xffffffffu, bm[i], 2));
    }
    float alpha[2], mn[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mn[i] = fmaxf(m[i], bm[i]);
      alpha[i] = (mn[i] == -INFINITY) ? 1.f : exp2f((m[i] - mn[i]) * LOG2E);
      m[i] = mn[i];
    }
    // P = exp(S - m); row sums in fp32 of the unrounded p; P rounded to bf16 for P V
    uint32_t pf[KB / 16][4];
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < KB / 8; ++j) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ri = e >> 1;
        p[e] = (s[j][e] == -INFINITY) ? 0.f : exp2f((s[j][e] - mn[ri]) * LOG2E);
        ls[ri] += p[e];
      }
      pf[j >> 1][(j & 1) * 2 + 0] = pack_bf2(p[0], p[1]);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_bf2(p[2], p[3]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {  // a row's 64 probabilities are spread over the 4 lanes of its quad
      ls[i] += __shfl_xor_sync(0xffffffffu, ls[i], 1);
      ls[i] += __shfl_xor_sync(0xffffffffu, ls[i], 2);
      l[i] = l[i] * alpha[i] + ls[i];
    }
#pragma unroll
    for (int j = 0; j < DT; ++j) { o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1]; }
    // O += P V : k-steps of 16 keys, n-tiles of 8 output columns (two per ldmatrix.x4.trans)
#pragma unroll
    for (int kk = 0; kk < KB / 16; ++kk) {
#pragma unroll
      for (int jd = 0; jd < DT; jd += 2) {
        uint32_t b0, b1, b2, b3;
        const int vr = kk * 16 + (lane & 15);
        const int vc = jd * 8 + ((lane >> 4) << 3);
        ldmatrix_x4_trans(b0, b1, b2, b3, (uint32_t)__cvta_generic_to_shared(&sv[vr * LD + vc]));
        mma_bf16_16816(o[jd], pf[kk], b0, b1);
        mma_bf16_16816(o[jd + 1], pf[kk], b2, b3);
      }
    }
  }

  // self key of candidate rows: one more online-softmax step with a per-row dot product
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const bool is_cand = segq[i] == -1;  // warp-uniform per quad only, so every lane runs the shuffles
    float dot = 0.f;
    const long long tok = (long long)b * T + (rq[i] < T ? rq[i] : 0);
    const bf16* kp = a.k + tok * a.k_tok_stride + (long long)hk * a.k_head_stride;
    if (is_cand) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const float2 qa = unpack_bf2(qf[ks][i]), qb = unpack_bf2(qf[ks][i + 2]);
        const float2 ka = unpack_bf2(*reinterpret_cast<const uint32_t*>(kp + ks * 16 + 2 * t4));
        const float2 kb = unpack_bf2(*reinterpret_cast<const uint32_t*>(kp + ks * 16 + 2 * t4 + 8));
        dot += qa.x * ka.x + qa.y * ka.y + qb.x * kb.x + qb.y * kb.y;
      }
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    if (is_cand) {
      const float sv_ = cap_logit(dot * a.sm_scale, a.cap, a.cap_method);
      const float mn = fmaxf(m[i], sv_);
      const float alpha = (m[i] == -INFINITY) ? 0.f : exp2f((m[i] - mn) * LOG2E);
      const float p = exp2f((sv_ - mn) * LOG2E);
      const float pr = round_bf(p);
      l[i] = l[i] * alpha + p;
      m[i] = mn;
      const bf16* vp = a.v + tok * a.v_tok_stride + (long long)hk * a.v_head_stride;
#pragma unroll
      for (int j = 0; j < DT; ++j) {
        const float2 vv = unpack_bf2(*reinterpret_cast<const uint32_t*>(vp + j * 8 + 2 * t4));
        o[j][2 * i + 0] = o[j][2 * i + 0] * alpha + pr * vv.x;
        o[j][2 * i + 1] = o[j][2 * i + 1] * alpha + pr * vv.y;
      }
    }
  }

  // normalise and store (rows with no allowed key: l == 0 -> zeros)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (rq[i] >= T) continue;
    const float inv = (l[i] == 0.f) ? 0.f : 1.0f / l[i];
    bf16* op = a.out + (((long long)b * T + rq[i]) * a.Hq + h) * DH;
#pragma unroll
    for (int j = 0; j < DT; ++j)
      *reinterpret_cast<uint32_t*>(op + j * 8 + 2 * t4) = pack_bf2(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
  }
}

}  // namespace

phx_status ranker_attention_launch(const AttnArgs& a, cudaStream_t stream, std::string& err) {
  if (a.Hq % a.Hkv != 0) { err = "attention: Hq must be a multiple of Hkv"; return PHX_E_ARG; }
  if (a.B == 0 || a.T == 0) return PHX_OK;
  if (a.B > 65535 || a.Hq > 65535) { err = "attention: batch or head count too large for one launch"; return PHX_E_CAPACITY; }
  dim3 grid((a.T + QROWS - 1) / QROWS, a.Hq, a.B);
  switch (a.dh) {
    case 32: ranker_attention_kernel<32><<<grid, ATT_THREADS, 0, stream>>>(a); break;
    case 64: ranker_attention_kernel<64><<<grid, ATT_THREADS, 0, stream>>>(a); break;
    case 128: ranker_attention_kernel<128><<<grid, ATT_THREADS, 0, stream>>>(a); break;
    default: err = "attention: head dim must be 32, 64 or 128"; return PHX_E_ARG;
  }
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

}  // namespace phx
