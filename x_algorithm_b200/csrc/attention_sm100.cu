// Candidate-isolated ("ranker") attention on Blackwell tensor cores (tcgen05 + TMEM + TMA); same semantics as
// attention.cu (mask: phoenix/xrex/pallas/ranker_attention_utils.py:16-56; softmax and P rounding:
// phoenix/xrex/pallas/ranker_attention_v2.py:113-148, 183).
//
// One CTA = 128 query rows of one (batch, head), 192 threads:
//   warp 0      TMA producer: the Q tile once, then per key block the K tile and the V tile (3-D tensor maps over
//               [batch][token][column]: rows past the request's last token are zero-filled, never the next request's)
//   warp 1      MMA issuer: S = Q K^T into TMEM (M=128, N=keys of the block), later O += P V with P read from shared
//               memory (K-major) and V as an MN-major operand straight from its row-major tile
//   warps 2-5   softmax: thread = query row; S row from TMEM, mask / max / exp2 / row sum in registers, P rounded to
//               bf16 into swizzled shared memory, O rescaled in TMEM when the running max moved; at the end the
//               candidate's self key is folded in with a per-row dot product, O is normalised, staged in shared
//               memory and written with TMA stores
// Only history keys are ever multiplied: the candidate x candidate block does not exist in this kernel.
// Waits are bounded; when one runs out the flag is raised and every later wait returns at once, so all roles
// drain through the same control flow (no thread is left at a barrier) and the host reports PHX_E_TIMEOUT.
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace phx {
namespace {

using namespace sm100;

constexpr int QT = 128;            // query rows per CTA
constexpr int A_THREADS = 192;
constexpr int SLAB = QT * 128;     // bytes of one [128 rows x 64 bf16] swizzled tile
constexpr int TC_MAX_BLOCKS = 256; // key blocks whose validity words fit the CTA's table

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float capped_log2(float s, float sm_scale, float cap, int method) {
  float v = s * sm_scale;
  if (method == 1) v = v / (1.0f + fabsf(v) / cap);
  else if (method == 2) v = cap * tanhf(v / cap);
  return v * 1.4426950408889634f;
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void bar_sync_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void st_shared_16(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

struct AttnTcArgs {
  const bf16* q; const bf16* k; const bf16* v;          // for the per-row self term (plain loads)
  bf16* out;                                            // [B*T][Hq][dh], for kernels that store rows directly
  long long q_tok_stride, k_tok_stride, v_tok_stride;
  int q_head_stride, k_head_stride, v_head_stride;
  const int* seg;
  int B, T, Hq, Hkv, hist_len;
  float sm_scale, cap;
  int cap_method;
  int* err_flag;
};

// D[tmem] (+)= A[tmem] * B[smem desc]: the A operand (bf16 pairs, one row per lane) comes from tensor memory
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
// 32 registers per thread -> 32 lanes x 32 columns, completion left to a later tcgen05.wait::st
__device__ __forceinline__ void tmem_st32_nowait(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// 16 registers per thread -> 32 lanes x 16 columns
__device__ __forceinline__ void tmem_st16_nowait(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// Wait for the tensor-memory loads in flight.  The 32 registers of the load that is about to be used are operands of
// the statement, so that no use of them can be scheduled in front of it (another load may have been issued since and
// other work done in between: the wait is the only thing that orders the registers' arrival).
__device__ __forceinline__ void tmem_ld_wait_on(float (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+f"(r[0]), "+f"(r[1]), "+f"(r[2]), "+f"(r[3]), "+f"(r[4]), "+f"(r[5]), "+f"(r[6]), "+f"(r[7]),
                 "+f"(r[8]), "+f"(r[9]), "+f"(r[10]), "+f"(r[11]), "+f"(r[12]), "+f"(r[13]), "+f"(r[14]), "+f"(r[15]),
                 "+f"(r[16]), "+f"(r[17]), "+f"(r[18]), "+f"(r[19]), "+f"(r[20]), "+f"(r[21]), "+f"(r[22]), "+f"(r[23]),
                 "+f"(r[24]), "+f"(r[25]), "+f"(r[26]), "+f"(r[27]), "+f"(r[28]), "+f"(r[29]), "+f"(r[30]), "+f"(r[31])
               :: "memory");
}

template <int DH, bool CAP>
__global__ void __launch_bounds__(A_THREADS, 2)
ranker_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                           AttnTcArgs a) {
  constexpr int KBLK = (DH == 64) ? 128 : 64;   // keys per block (keeps shared memory at 80 KB: two CTAs per SM)
  constexpr int DCH = DH / 64;                  // 64-column chunks of the head dim
  // S is double-buffered in TMEM (and K in shared memory): S of block j+1 is computed while the softmax warps are
  // still on block j, so the tensor pipe and the softmax overlap inside one CTA.  KBLK <= 64 or two S buffers of
  // 128 columns would not fit next to O in the CTA's 256 columns; at head dim 64 (KBLK 128) S stays single.
  constexpr int NSB = (KBLK <= 64) ? 2 : 1;     // S buffers (TMEM) = K buffers (shared memory)
  constexpr uint32_t TM_S = 0, TM_O = 128;      // TMEM columns of S (NSB x KBLK) and O
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base;                               // DCH x [128 x 128 B]; reused to stage the output
  const uint32_t sK = sQ + DCH * SLAB;                    // NSB x DCH x [KBLK x 128 B]
  const uint32_t sV = sK + NSB * DCH * KBLK * 128;        // 2 x DCH x [KBLK x 128 B]
  const uint32_t sMask = sV + 2 * DCH * KBLK * 128;       // [TC_MAX_BLOCKS][4] key-validity words
  const uint32_t bars = sMask + TC_MAX_BLOCKS * 16;
  const uint32_t q_full = bars, p_ready = bars + 24, o_done = bars + 32, tmem_slot = bars + 88;
  auto v_full = [&](int i) { return bars + (i ? 96u : 8u); };
  auto v_empty = [&](int i) { return bars + (i ? 104u : 16u); };
  auto k_full = [&](int i) { return bars + 40u + 8u * i; };
  auto k_empty = [&](int i) { return bars + 56u + 8u * i; };
  auto s_full = [&](int i) { return bars + 72u + 8u * i; };
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  uint32_t* mask_words = reinterpret_cast<uint32_t*>(smem_raw + (sMask - smem_u32(smem_raw)));

  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * QT;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = a.T;
  const int n_hist = a.hist_len < T ? a.hist_len : T;
  const int n_blocks = (n_hist + KBLK - 1) / KBLK;
  volatile int* verr = a.err_flag;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(p_ready, 128); mbar_init(o_done, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(k_full(i), 1); mbar_init(k_empty(i), 1); mbar_init(s_full(i), 1); mbar_init(v_full(i), 1); mbar_init(v_empty(i), 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_expect_tx(q_full, DCH * SLAB);
      for (int c = 0; c < DCH; ++c) tma_load_3d(sQ + c * SLAB, &map_q, q_full, h * a.q_head_stride + c * 64, q0, b);
      auto load_k = [&](int j) {   // K block j into buffer j % NSB, once S of block j - NSB has been computed
        const int kb = j % NSB; const uint32_t use = (uint32_t)(j / NSB);
        mbar_wait(k_empty(kb), (use & 1) ^ 1, verr);
        mbar_expect_tx(k_full(kb), DCH * KBLK * 128);
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sK + (kb * DCH + c) * KBLK * 128, &map_k, k_full(kb), hk * a.k_head_stride + c * 64, j * KBLK, b);
      };
      for (int j = 0; j < NSB - 1 && j < n_blocks; ++j) load_k(j);
      for (int j = 0; j < n_blocks; ++j) {
        if (j + NSB - 1 < n_blocks) load_k(j + NSB - 1);
        const int vb = j & 1;                           // V is double-buffered: block j + 1 arrives under P V of block j
        mbar_wait(v_empty(vb), (uint32_t)((j >> 1) & 1) ^ 1u, verr);
        mbar_expect_tx(v_full(vb), DCH * KBLK * 128);
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sV + (vb * DCH + c) * KBLK * 128, &map_v, v_full(vb), hk * a.v_head_stride + c * 64, j * KBLK, b);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(QT, KBLK);
      constexpr uint32_t idesc_o = make_idesc_b_mn(QT, DH);
      mbar_wait(q_full, 0, verr);
      auto issue_s = [&](int j) {   // S(j) = Q K(j)^T into S buffer j % NSB
        const int kb = j % NSB; const uint32_t use = (uint32_t)(j / NSB);
        mbar_wait(k_full(kb), use & 1, verr);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          const uint64_t qd = make_smem_desc(sQ + c * SLAB), kd = make_smem_desc(sK + (kb * DCH + c) * KBLK * 128);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem + TM_S + kb * KBLK, qd + (uint64_t)(k * 2), kd + (uint64_t)(k * 2), idesc_s, (c | k) != 0);
        }
        umma_commit(k_empty(kb));
        umma_commit(s_full(kb));
      };
      for (int j = 0; j < NSB - 1 && j < n_blocks; ++j) issue_s(j);
      for (int j = 0; j < n_blocks; ++j) {
        const uint32_t ph = (uint32_t)(j & 1);
        // the S buffer of block j + NSB - 1 was last read by the softmax of block j - 1, whose P has been awaited below
        if (j + NSB - 1 < n_blocks) issue_s(j + NSB - 1);
        const int vb = j & 1;
        mbar_wait(p_ready, ph, verr);
        mbar_wait(v_full(vb), (uint32_t)((j >> 1) & 1), verr);
        tc_fence_after();
        // P sits in tensor memory, as bf16 pairs over the first KBLK / 2 columns of the S buffer it was computed from
        // (16 keys = 8 columns per step); that buffer is overwritten by S of block j + NSB, issued after this product
#pragma unroll
        for (int kk = 0; kk < KBLK / 16; ++kk) {
          const uint64_t vd = make_smem_desc_mn(sV + vb * DCH * KBLK * 128 + kk * 16 * 128, KBLK * 128, 1024);
          umma_bf16_ts(tmem + TM_O, tmem + TM_S + (j % NSB) * KBLK + kk * 8, vd, idesc_o, (j | kk) != 0);
        }
        umma_commit(v_empty(vb));
        umma_commit(o_done);
      }
    }
  } else {
    // ---------------- softmax / epilogue (warps 2..5, thread = query row) ----------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int sw = r & 7;
    const int row = q0 + r;
    const long long tok0 = (long long)b * T;
    const int segq = (row < T) ? a.seg[tok0 + row] : 0;
    const uint32_t lane_base = ((uint32_t)(quad * 32) << 16);
    const float csc = CAP ? 1.0f : a.sm_scale * 1.4426950408889634f;
    float m = -INFINITY, l = 0.f;

    // validity of every history key, once per CTA (thread r looks at key r of each block; the loads of all blocks are
    // in flight together instead of one exposed round trip per block)
    for (int j = 0; j < n_blocks; ++j) {
      const int key = j * KBLK + r;
      const bool ok = (r < KBLK) && (key < n_hist) && (a.seg[tok0 + key] == 1);
      const uint32_t word = __ballot_sync(0xffffffffu, ok);
      if (lane == 0) mask_words[j * 4 + quad] = word;
    }
    bar_sync_128();

    for (int j = 0; j < n_blocks; ++j) {
      const uint32_t ph = (uint32_t)(j & 1);
      uint32_t kmask[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) kmask[w] = mask_words[j * 4 + w];
      bool all_ok = true;
#pragma unroll
      for (int w = 0; w < KBLK / 32; ++w) all_ok = all_ok && (kmask[w] == 0xffffffffu);

      mbar_wait(s_full(j % NSB), (uint32_t)((j / NSB) & 1), verr);
      tc_fence_after();
      float s[KBLK];
#pragma unroll
      for (int c = 0; c < KBLK / 32; ++c) tmem_ld32_nowait(tmem + TM_S + (j % NSB) * KBLK + lane_base + c * 32, reinterpret_cast<uint32_t*>(s) + c * 32);
      tmem_ld_wait();
      if (CAP) {
#pragma unroll
        for (int k = 0; k < KBLK; ++k) s[k] = capped_log2(s[k], a.sm_scale, a.cap, a.cap_method);
      }
      if (!all_ok) {
#pragma unroll
        for (int k = 0; k < KBLK; ++k)
          if (!((kmask[k >> 5] >> (k & 31)) & 1u)) s[k] = -INFINITY;
      }
      float bm;
      {
        float b4[4] = {s[0], s[1], s[2], s[3]};   // four chains of three-input max
#pragma unroll
        for (int k = 4; k + 7 < KBLK + 4 && k + 7 < KBLK; k += 8) {
          b4[0] = max3f(b4[0], s[k], s[k + 1]); b4[1] = max3f(b4[1], s[k + 2], s[k + 3]);
          b4[2] = max3f(b4[2], s[k + 4], s[k + 5]); b4[3] = max3f(b4[3], s[k + 6], s[k + 7]);
        }
        bm = fmaxf(max3f(b4[0], b4[1], b4[2]), b4[3]);
#pragma unroll
        for (int k = KBLK - 4; k < KBLK; ++k) bm = fmaxf(bm, s[k]);   // the tail the 8-wide loop leaves (4 elements)
      }
      // The reference point of the exponentials only has to bound them, not equal the running maximum: it moves
      // when the maximum has grown by more than 2^8 since it was set (P stays below 256, exact in bf16 up to the same
      // power of two), which spares the rescaling of O in tensor memory for almost every block.
      const float m_true = fmaxf(m, bm * csc);
      const bool move = __any_sync(0xffffffffu, m_true > m + 8.0f || (m == -INFINITY && m_true != -INFINITY));
      const float m_new = move ? m_true : m;
      const float mns = (m_new == -INFINITY) ? 0.f : m_new;   // finite stand-in while nothing is allowed yet
      const float alpha = ex2f(m - mns);                      // -inf - finite -> 0; unmoved: 1
      m = m_new;
      float ls;
      {
        const float2 c2 = make_float2(csc, csc), n2 = make_float2(-mns, -mns);
        float2 acc2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int k = 0; k < KBLK; k += 2) {   // packed fp32: two columns per instruction; masked: 2^-inf = 0
          const float2 e = __ffma2_rn(make_float2(s[k], s[k + 1]), c2, n2);
          s[k] = ex2f(e.x); s[k + 1] = ex2f(e.y);
          acc2[(k >> 1) & 1] = __fadd2_rn(acc2[(k >> 1) & 1], make_float2(s[k], s[k + 1]));
        }
        ls = (acc2[0].x + acc2[0].y) + (acc2[1].x + acc2[1].y);
      }
      l = l * alpha + ls;

      if (j > 0) {
        // O of the previous blocks must be complete (and P's previous contents consumed) before it is rescaled
        mbar_wait(o_done, ph ^ 1, verr);
        tc_fence_after();
        const bool need = __any_sync(0xffffffffu, alpha != 1.0f);
        if (need) {
#pragma unroll
          for (int c = 0; c < DH / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem + TM_O + lane_base + c * 32, o);
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * alpha);
            tmem_st32(tmem + TM_O + lane_base + c * 32, o);
          }
        }
      }
      // P (bf16 pairs) back into tensor memory, over the first KBLK / 2 columns of this block's S buffer (the whole
      // row of S is in registers by now): the second MMA takes its A operand from there
      {
        uint32_t pw[KBLK / 2];
#pragma unroll
        for (int k = 0; k < KBLK / 2; ++k) pw[k] = pack_bf2(s[2 * k], s[2 * k + 1]);
#pragma unroll
        for (int c = 0; c < KBLK / 64; ++c) tmem_st32_nowait(tmem + TM_S + (j % NSB) * KBLK + lane_base + c * 32, pw + c * 32);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      tc_fence_before();
      mbar_arrive(p_ready);
    }

    // ---- epilogue: O row, self key of a candidate, normalise, stage, TMA store --------------------------------
    float o[DH];
    if (n_blocks > 0) {
      mbar_wait(o_done, (uint32_t)((n_blocks - 1) & 1), verr);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) tmem_ld32(tmem + TM_O + lane_base + c * 32, reinterpret_cast<uint32_t*>(o) + c * 32);
    } else {
#pragma unroll
      for (int k = 0; k < DH; ++k) o[k] = 0.f;
    }
    if (segq == -1) {
      const long long tok = tok0 + row;
      const uint4* qp = reinterpret_cast<const uint4*>(a.q + tok * a.q_tok_stride + (long long)h * a.q_head_stride);
      const uint4* kp = reinterpret_cast<const uint4*>(a.k + tok * a.k_tok_stride + (long long)hk * a.k_head_stride);
      const uint4* vp = reinterpret_cast<const uint4*>(a.v + tok * a.v_tok_stride + (long long)hk * a.v_head_stride);
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < DH / 8; ++c) {
        const uint4 qa = __ldg(qp + c), ka = __ldg(kp + c);
        const float2 q0f = unpack_bf2(qa.x), q1f = unpack_bf2(qa.y), q2f = unpack_bf2(qa.z), q3f = unpack_bf2(qa.w);
        const float2 k0f = unpack_bf2(ka.x), k1f = unpack_bf2(ka.y), k2f = unpack_bf2(ka.z), k3f = unpack_bf2(ka.w);
        dot += q0f.x * k0f.x + q0f.y * k0f.y + q1f.x * k1f.x + q1f.y * k1f.y + q2f.x * k2f.x + q2f.y * k2f.y + q3f.x * k3f.x + q3f.y * k3f.y;
      }
      const float sv = CAP ? capped_log2(dot, a.sm_scale, a.cap, a.cap_method) : dot * csc;
      const float mn = fmaxf(m, sv);
      const float alpha = ex2f(m - mn);           // no history: 2^-inf = 0
      const float p = ex2f(sv - mn);
      const float pr = round_bf(p);
      l = l * alpha + p;
#pragma unroll
      for (int c = 0; c < DH / 8; ++c) {
        const uint4 va = __ldg(vp + c);
        const float2 v0 = unpack_bf2(va.x), v1 = unpack_bf2(va.y), v2 = unpack_bf2(va.z), v3 = unpack_bf2(va.w);
        o[c * 8 + 0] = o[c * 8 + 0] * alpha + pr * v0.x; o[c * 8 + 1] = o[c * 8 + 1] * alpha + pr * v0.y;
        o[c * 8 + 2] = o[c * 8 + 2] * alpha + pr * v1.x; o[c * 8 + 3] = o[c * 8 + 3] * alpha + pr * v1.y;
        o[c * 8 + 4] = o[c * 8 + 4] * alpha + pr * v2.x; o[c * 8 + 5] = o[c * 8 + 5] * alpha + pr * v2.y;
        o[c * 8 + 6] = o[c * 8 + 6] * alpha + pr * v3.x; o[c * 8 + 7] = o[c * 8 + 7] * alpha + pr * v3.y;
      }
    }
    const float inv = (l == 0.f || segq == 0) ? 0.f : 1.0f / l;   // padded rows, rows with no allowed key -> zeros
#pragma unroll
    for (int c = 0; c < DH / 8; ++c) {
      uint4 w;
      w.x = pack_bf2(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv); w.y = pack_bf2(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
      w.z = pack_bf2(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv); w.w = pack_bf2(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
      st_shared_16(sQ + (c >> 3) * SLAB + r * 128 + ((uint32_t)((c & 7) ^ sw) << 4), w);   // Q is no longer needed
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    bar_sync_128();
    if (warp == 2 && lane == 0) {
      for (int c = 0; c < DCH; ++c) tma_store_3d(&map_o, sQ + c * SLAB, h * DH + c * 64, q0, b);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  }

  if (*verr != 0) __nanosleep(1000000);  // error path: let in-flight bulk copies land before the CTA retires
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ---- resident-history variant -----------------------------------------------------------------------------------
// History of at most 128 keys, head dim 64 (the ranking trunk's shape): K and V of the (batch, head) are loaded once
// and stay in shared memory while the CTA walks over all of the request's query tiles.  Q tiles are double-buffered
// (the producer runs ahead), O is double-buffered in TMEM, so S = Q K^T of tile t+1 is issued while the softmax
// warps still normalise tile t; output rows go straight from registers to global memory (128 contiguous bytes per
// thread), and the rows a candidate needs for its self key are requested one tile ahead.
__global__ void __launch_bounds__(A_THREADS, 2)
ranker_attention_resident_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                                 AttnTcArgs a, int cap_on) {
  constexpr int DH = 64, KBLK = 128;
  constexpr uint32_t TM_S = 0, TM_O = 128;      // O buffers at columns 128 and 192
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base;                     // 2 x [128 x 128 B]
  const uint32_t sK = sQ + 2 * SLAB;            // [128 x 128 B]
  const uint32_t sV = sK + SLAB;                // [128 x 128 B]
  const uint32_t sP = sV + SLAB;                // 2 x [128 x 128 B]
  const uint32_t sMask = sP + 2 * SLAB;
  const uint32_t bars = sMask + 64;
  auto q_full = [&](int i) { return bars + 8u * i; };
  auto q_free = [&](int i) { return bars + 16u + 8u * i; };
  const uint32_t kv_full = bars + 32, s_full = bars + 40, p_ready = bars + 48, o_done = bars + 56, tmem_slot = bars + 64;
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  uint32_t* mask_words = reinterpret_cast<uint32_t*>(smem_raw + (sMask - smem_u32(smem_raw)));

  const int b = blockIdx.z, h = blockIdx.y;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T = a.T;
  const int n_hist = a.hist_len < T ? a.hist_len : T;
  const int n_tiles = (T + QT - 1) / QT;
  volatile int* verr = a.err_flag;

  if (threadIdx.x == 0) {
    // a Q buffer is free once S has been computed from it (commit) and the 128 softmax threads have read their rows
    for (int i = 0; i < 2; ++i) { mbar_init(q_full(i), 1); mbar_init(q_free(i), 129); }
    mbar_init(kv_full, 1); mbar_init(s_full, 1); mbar_init(p_ready, 128); mbar_init(o_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * SLAB);
      tma_load_3d(sK, &map_k, kv_full, hk * a.k_head_stride, 0, b);
      tma_load_3d(sV, &map_v, kv_full, hk * a.v_head_stride, 0, b);
      for (int t = 0; t < n_tiles; ++t) {
        const int bq = t & 1;
        mbar_wait(q_free(bq), (uint32_t)(((t >> 1) & 1) ^ 1), verr);
        mbar_expect_tx(q_full(bq), SLAB);
        tma_load_3d(sQ + bq * SLAB, &map_q, q_full(bq), h * a.q_head_stride, t * QT, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(QT, KBLK);
      constexpr uint32_t idesc_o = make_idesc_b_mn(QT, DH);
      mbar_wait(kv_full, 0, verr);
      for (int t = 0; t < n_tiles; ++t) {
        const int bq = t & 1;
        const uint32_t ph = (uint32_t)(t & 1);
        mbar_wait(q_full(bq), (uint32_t)((t >> 1) & 1), verr);
        tc_fence_after();
        const uint64_t qd = make_smem_desc(sQ + bq * SLAB), kd = make_smem_desc(sK);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + TM_S, qd + (uint64_t)(k * 2), kd + (uint64_t)(k * 2), idesc_s, k != 0);
        umma_commit(s_full);
        umma_commit(q_free(bq));          // the Q buffer is free as soon as S has been computed
        mbar_wait(p_ready, ph, verr);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < KBLK / 16; ++kk) {
          const uint64_t pd = make_smem_desc(sP + (kk >> 2) * SLAB) + (uint64_t)((kk & 3) * 2);
          const uint64_t vd = make_smem_desc_mn(sV + kk * 16 * 128, KBLK * 128, 1024);
          umma_bf16(tmem + TM_O + bq * DH, pd, vd, idesc_o, kk != 0);
        }
        umma_commit(o_done);
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int sw = r & 7;
    const long long tok0 = (long long)b * T;
    const uint32_t lane_base = ((uint32_t)(quad * 32) << 16);
    const float csc = cap_on ? 1.0f : a.sm_scale * 1.4426950408889634f;
    // key validity, the same for every tile of the request
    {
      const bool ok = (r < n_hist) && (a.seg[tok0 + r] == 1);
      const uint32_t word = __ballot_sync(0xffffffffu, ok);
      if (lane == 0) mask_words[quad] = word;
    }
    bar_sync_128();
    uint32_t kmask[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) kmask[w] = mask_words[w];
    const bool all_ok = (kmask[0] & kmask[1] & kmask[2] & kmask[3]) == 0xffffffffu;

    // Per-row work for a candidate's self key needs the row's own q, k and v.  Its k and v rows come from HBM, so
    // they are requested one tile ahead: k(t+1) at the start of tile t (used after tile t's softmax, when the dot
    // product for tile t+1 is formed against the Q row already sitting in the Q buffer), v(t+1) at the end of tile t.
    const bf16* kbase = a.k + (long long)hk * a.k_head_stride;
    const bf16* vbase = a.v + (long long)hk * a.v_head_stride;
    auto seg_of = [&](int t) { const int row = t * QT + r; return (row < T) ? a.seg[tok0 + row] : 0; };
    auto tok_of = [&](int t) { const int row = t * QT + r; return tok0 + (row < T ? row : 0); };
    auto load_row = [&](const bf16* base, long long stride, int t, bool on, uint4 (&dst)[DH / 8]) {
      if (on) {
        const uint4* p = reinterpret_cast<const uint4*>(base + tok_of(t) * stride);
#pragma unroll
        for (int c = 0; c < DH / 8; ++c) dst[c] = __ldg(p + c);
      }
    };
    // q(t) . k(t) for this row, q from the (swizzled) Q buffer; every thread then lets go of the buffer
    auto self_dot = [&](int t, bool on, const uint4 (&krow)[DH / 8]) {
      const int bq = t & 1;
      mbar_wait(q_full(bq), (uint32_t)((t >> 1) & 1), verr);
      float dot = 0.f;
      if (on) {
        float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < DH / 8; ++c) {
          uint4 qa;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(qa.x), "=r"(qa.y), "=r"(qa.z), "=r"(qa.w)
                       : "r"(sQ + bq * SLAB + r * 128 + ((uint32_t)(c ^ sw) << 4)));
          const uint4 ka = krow[c];
          const float2 q0f = unpack_bf2(qa.x), q1f = unpack_bf2(qa.y), q2f = unpack_bf2(qa.z), q3f = unpack_bf2(qa.w);
          const float2 k0f = unpack_bf2(ka.x), k1f = unpack_bf2(ka.y), k2f = unpack_bf2(ka.z), k3f = unpack_bf2(ka.w);
          d4[0] += q0f.x * k0f.x + q0f.y * k0f.y; d4[1] += q1f.x * k1f.x + q1f.y * k1f.y;
          d4[2] += q2f.x * k2f.x + q2f.y * k2f.y; d4[3] += q3f.x * k3f.x + q3f.y * k3f.y;
        }
        dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
      }
      mbar_arrive(q_free(bq));
      return cap_on ? capped_log2(dot, a.sm_scale, a.cap, a.cap_method) : dot * csc;
    };
    // one 64-key half of the S row, capped and masked, into registers
    auto load_s_half = [&](int c, float (&sv)[64]) {
      tmem_ld32_nowait(tmem + TM_S + lane_base + c * 64, reinterpret_cast<uint32_t*>(sv));
      tmem_ld32_nowait(tmem + TM_S + lane_base + c * 64 + 32, reinterpret_cast<uint32_t*>(sv) + 32);
      tmem_ld_wait();
      if (cap_on) {
#pragma unroll
        for (int k = 0; k < 64; ++k) sv[k] = capped_log2(sv[k], a.sm_scale, a.cap, a.cap_method);
      }
      if (!all_ok) {
#pragma unroll
        for (int k = 0; k < 64; ++k)
          if (!((kmask[c * 2 + (k >> 5)] >> (k & 31)) & 1u)) sv[k] = -INFINITY;
      }
    };

    uint4 krow[DH / 8], vrow[DH / 8];
    int segq = seg_of(0);
    int seg_next = (1 < n_tiles) ? seg_of(1) : 0;
    load_row(kbase, a.k_tok_stride, 0, segq == -1, krow);
    load_row(vbase, a.v_tok_stride, 0, segq == -1, vrow);
    float self_logit = self_dot(0, segq == -1, krow);

    for (int t = 0; t < n_tiles; ++t) {
      const int bq = t & 1;
      const uint32_t ph = (uint32_t)(t & 1);
      const int row = t * QT + r;
      const bool more = (t + 1 < n_tiles);
      const int seg_next2 = (t + 2 < n_tiles) ? seg_of(t + 2) : 0;   // two tiles ahead: it gates the loads issued next tile
      if (more) load_row(kbase, a.k_tok_stride, t + 1, seg_next == -1, krow);

      mbar_wait(s_full, ph, verr);
      tc_fence_after();
      // pass 1: row maximum (S is read twice, 64 keys at a time, to keep the row out of the register file)
      float bm = -INFINITY;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float sv[64];
        load_s_half(c, sv);
        float b4[4] = {sv[0], sv[1], sv[2], sv[3]};   // four independent chains: the warp has little else to overlap with
#pragma unroll
        for (int k = 4; k < 64; ++k) b4[k & 3] = fmaxf(b4[k & 3], sv[k]);
        bm = fmaxf(bm, fmaxf(fmaxf(b4[0], b4[1]), fmaxf(b4[2], b4[3])));
      }
      float m = bm * csc;
      if (segq == -1) m = fmaxf(m, self_logit);          // the self key takes part in the row maximum right away
      const float mns = (m == -INFINITY) ? 0.f : m;
      // P's previous contents (tile t-1) must have been consumed by its P V product
      if (t > 0) mbar_wait(o_done, ph ^ 1, verr);
      // pass 2: probabilities, row sum, P in bf16 into the swizzled operand buffer
      float l = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float sv[64];
        load_s_half(c, sv);
#pragma unroll
        for (int k = 0; k < 64; ++k) sv[k] = ex2f(fmaf(sv[k], csc, -mns));
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < 64; ++k) l4[k & 3] += sv[k];
        l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          uint4 o;
          o.x = pack_bf2(sv[cc * 8 + 0], sv[cc * 8 + 1]); o.y = pack_bf2(sv[cc * 8 + 2], sv[cc * 8 + 3]);
          o.z = pack_bf2(sv[cc * 8 + 4], sv[cc * 8 + 5]); o.w = pack_bf2(sv[cc * 8 + 6], sv[cc * 8 + 7]);
          st_shared_16(sP + c * SLAB + r * 128 + ((uint32_t)(cc ^ sw) << 4), o);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(p_ready);

      // while the P V product runs: the self logit of the next tile (its k row was requested at the top)
      float self_next = 0.f;
      if (more) self_next = self_dot(t + 1, seg_next == -1, krow);

      // ---- epilogue of this tile ----
      float p_self = 0.f;
      if (segq == -1) { p_self = ex2f(self_logit - mns); l += p_self; }
      const float pr = round_bf(p_self);
      mbar_wait(o_done, ph, verr);
      tc_fence_after();
      float o[DH];
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) tmem_ld32(tmem + TM_O + bq * DH + lane_base + c * 32, reinterpret_cast<uint32_t*>(o) + c * 32);
      const float inv = (l == 0.f || segq == 0) ? 0.f : 1.0f / l;
      // the thread's output row is 128 contiguous bytes: four 32-byte stores, no staging
      bf16* orow = a.out + ((tok0 + row) * a.Hq + h) * DH;
#pragma unroll
      for (int c2 = 0; c2 < DH / 16; ++c2) {
        uint32_t w[8];
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          const int c = c2 * 2 + hc;
          if (segq == -1) {
            const float2 v0 = unpack_bf2(vrow[c].x), v1 = unpack_bf2(vrow[c].y), v2 = unpack_bf2(vrow[c].z), v3 = unpack_bf2(vrow[c].w);
            o[c * 8 + 0] += pr * v0.x; o[c * 8 + 1] += pr * v0.y; o[c * 8 + 2] += pr * v1.x; o[c * 8 + 3] += pr * v1.y;
            o[c * 8 + 4] += pr * v2.x; o[c * 8 + 5] += pr * v2.y; o[c * 8 + 6] += pr * v3.x; o[c * 8 + 7] += pr * v3.y;
          }
          w[hc * 4 + 0] = pack_bf2(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv); w[hc * 4 + 1] = pack_bf2(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
          w[hc * 4 + 2] = pack_bf2(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv); w[hc * 4 + 3] = pack_bf2(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
        }
        if (row < T)
          asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                       ::"l"(orow + c2 * 16), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
      }
      // next tile's v row: a whole tile to arrive
      if (more) load_row(vbase, a.v_tok_stride, t + 1, seg_next == -1, vrow);
      segq = seg_next;
      seg_next = seg_next2;
      self_logit = self_next;
    }
  }

  if (*verr != 0) __nanosleep(1000000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ---- resident history, two softmax warpgroups (the ranking trunk's shape at throughput batch sizes) ----------------
// Head dim 64, at most 128 history keys.  A persistent CTA (one per SM, 352 threads) walks over (batch, head) items;
// per item the history K and V tiles are loaded once by TMA (double-buffered across items, so the next item's tiles
// arrive while the current one is still being worked on) and every 128-row query tile of the request streams through
// a three-deep ring of stages.  A stage holds the tile's Q rows and, for a candidate tile, the same rows of K and V:
// everything a tile reads from global memory arrives by bulk copies, and its output leaves the same way (the O rows
// are staged in the stage's Q slab, which the tensor core has long finished with, and a store warp hands them to TMA
// and releases the stage).  Two softmax warpgroups take alternate tiles, each with its own S and O accumulators in
// tensor memory (S0, S1 at columns 0 / 128, O0, O1 at 256 / 320): while one warpgroup exponentiates tile g, the MMA
// warp has already produced S of tile g+1 for the other, and P V of tile g runs under the other warpgroup's softmax.
// Thread = query row: the 128-key S row is read from tensor memory 64 keys at a time, once for the row maximum and
// once for the probabilities, which go straight back into tensor memory as bf16 pairs over the columns the row's S
// values came from; P V takes its A operand from there (no shared-memory round trip for P).
// The candidate x candidate block is never used as such: the tensor core forms Q Kc^T of the tile's own rows into a
// 128-column scratch (columns 384..511) and each thread picks its diagonal element - the candidate's score against
// its own key, one extra softmax term whose value row the thread reads from the stage.  Query tiles are taken from
// the history block and the candidate block separately, so the plain [B, T] token layout and the split layout (all
// history rows, then all candidate rows) differ only in the tensor maps' strides; candidate-only layers skip the
// history tiles.  All waits are bounded (sm100_ptx.cuh).
constexpr int PP_THREADS = 352;   // warp 0 TMA loads, warp 1 MMA, warps 2-5 / 6-9 softmax warpgroups 0 / 1, warp 10 TMA stores
constexpr int PP_NQ = 3;

struct PingArgs {
  const int* seg;
  int q_head_stride, k_head_stride, v_head_stride;
  int Hq, Hkv, n_hist, n_cand, n_items;
  long long hist_row0, hist_req_rows, cand_row0, cand_req_rows;   // token row of position 0 of request 0; rows per request
  int skip_hist;                                                  // 1: history rows are keys only (candidate-only layer)
  float sm_scale, cap;
  int cap_method;
  int* err_flag;
};

// the eight tensor maps of a launch: Q / K / V / out over the history block and over the candidate block
struct PingMaps { CUtensorMap qh, qc, kh, vh, kc, vc, oh, oc; };

template <bool CAP>
__global__ void __launch_bounds__(PP_THREADS, 1)
ranker_attention_pingpong_kernel(const __grid_constant__ PingMaps maps, PingArgs a) {
  constexpr int DH = 64;
  constexpr uint32_t TM_S = 0, TM_O = 256, TM_D = 384;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sKV = base;                       // 2 x (K [128 x 128 B], V [128 x 128 B])
  const uint32_t sQ = sKV + 4 * SLAB;              // PP_NQ stages x (Q, Kc, Vc), each [128 x 128 B]
  const uint32_t sMask = sQ + 3 * PP_NQ * SLAB;    // 2 warpgroups x 4 words
  const uint32_t bars = sMask + 64;
  auto kv_full = [&](int i) { return bars + 8u * i; };
  auto kv_free = [&](int i) { return bars + 16u + 8u * i; };
  auto q_full = [&](int i) { return bars + 32u + 8u * i; };
  auto q_free = [&](int i) { return bars + 56u + 8u * i; };
  auto s_full = [&](int i) { return bars + 80u + 8u * i; };
  auto p_ready = [&](int i) { return bars + 96u + 8u * i; };
  auto o_done = [&](int i) { return bars + 112u + 8u * i; };
  auto o_staged = [&](int i) { return bars + 128u + 8u * i; };
  const uint32_t d_free = bars + 144u;
  const uint32_t tmem_slot = bars + 152u;
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  uint32_t* mask_words = reinterpret_cast<uint32_t*>(smem_raw + (sMask - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* verr = a.err_flag;
  const int n_htiles = a.skip_hist ? 0 : (a.n_hist + QT - 1) / QT;      // 0 or 1
  const int n_ctiles = (a.n_cand + QT - 1) / QT;
  const int nt = n_htiles + n_ctiles;                                   // query tiles per item
  const int my_items = ((int)blockIdx.x < a.n_items) ? (a.n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int G = my_items * nt;                                          // tiles this CTA works through

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(kv_full(i), 1); mbar_init(kv_free(i), 1); mbar_init(s_full(i), 1); mbar_init(p_ready(i), 128);
      mbar_init(o_done(i), 1); mbar_init(o_staged(i), 128);
    }
    // a stage is free again once the tile's output rows, staged in its Q slab, have been read by the store
    for (int i = 0; i < PP_NQ; ++i) { mbar_init(q_full(i), 1); mbar_init(q_free(i), 1); }
    mbar_init(d_free, 128);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int g = 0;
      for (int li = 0; li < my_items; ++li) {
        const int it = (int)blockIdx.x + li * (int)gridDim.x;
        const int b = it / a.Hq, h = it % a.Hq, hk = h / (a.Hq / a.Hkv);
        const int kb = li & 1;
        mbar_wait(kv_free(kb), (uint32_t)(((li >> 1) & 1) ^ 1), verr);
        mbar_expect_tx(kv_full(kb), 2 * SLAB);
        tma_load_3d(sKV + (2 * kb) * SLAB, &maps.kh, kv_full(kb), hk * a.k_head_stride, 0, b);
        tma_load_3d(sKV + (2 * kb + 1) * SLAB, &maps.vh, kv_full(kb), hk * a.v_head_stride, 0, b);
        for (int ti = 0; ti < nt; ++ti, ++g) {
          const int st = g % PP_NQ;
          const uint32_t dst = sQ + 3 * st * SLAB;
          mbar_wait(q_free(st), (uint32_t)(((g / PP_NQ) & 1) ^ 1), verr);
          if (ti < n_htiles) {
            mbar_expect_tx(q_full(st), SLAB);
            tma_load_3d(dst, &maps.qh, q_full(st), h * a.q_head_stride, ti * QT, b);
          } else {
            const int r0 = (ti - n_htiles) * QT;
            mbar_expect_tx(q_full(st), 3 * SLAB);
            tma_load_3d(dst, &maps.qc, q_full(st), h * a.q_head_stride, r0, b);
            tma_load_3d(dst + SLAB, &maps.kc, q_full(st), hk * a.k_head_stride, r0, b);
            tma_load_3d(dst + 2 * SLAB, &maps.vc, q_full(st), hk * a.v_head_stride, r0, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(QT, 128);
      constexpr uint32_t idesc_o = make_idesc_b_mn(QT, DH);
      auto issue_pv = [&](int gp, int kbp, bool last_of_item) {      // O[w] = P[w] V for tile gp, P from tensor memory
        const int w = gp & 1;
        mbar_wait(p_ready(w), (uint32_t)((gp >> 1) & 1), verr);
        tc_fence_after();
        const uint32_t sV = sKV + (2 * kbp + 1) * SLAB;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {                             // 16 keys = 8 columns of bf16 pairs per step
          const uint64_t vd = make_smem_desc_mn(sV + kk * 16 * 128, 128 * 128, 1024);
          umma_bf16_ts(tmem + TM_O + w * DH, tmem + TM_S + w * 128 + kk * 8, vd, idesc_o, kk != 0);
        }
        umma_commit(o_done(w));
        if (last_of_item) umma_commit(kv_free(kbp));                 // every MMA that read this item's K / V is behind this point
      };
      int g = 0, prev_kb = 0, n_d = 0;
      bool prev_last = false;
      for (int li = 0; li < my_items; ++li) {
        const int kb = li & 1;
        mbar_wait(kv_full(kb), (uint32_t)((li >> 1) & 1), verr);
        for (int ti = 0; ti < nt; ++ti, ++g) {
          const int st = g % PP_NQ, w = g & 1;
          mbar_wait(q_full(st), (uint32_t)((g / PP_NQ) & 1), verr);
          tc_fence_after();
          // S[w] (and the P that overwrote part of it) is free: P V of tile g - 2 was issued before this point and the
          // tensor core runs its instructions in order
          const uint64_t qd = make_smem_desc(sQ + 3 * st * SLAB), kd = make_smem_desc(sKV + (2 * kb) * SLAB);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem + TM_S + w * 128, qd + (uint64_t)(k * 2), kd + (uint64_t)(k * 2), idesc_s, k != 0);
          if (ti >= n_htiles) {
            // the tile's rows against their own keys; the scratch is free once the previous candidate tile's warpgroup
            // has picked its diagonal
            mbar_wait(d_free, (uint32_t)((n_d & 1) ^ 1), verr);
            tc_fence_after();
            ++n_d;
            const uint64_t kcd = make_smem_desc(sQ + (3 * st + 1) * SLAB);
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_bf16(tmem + TM_D, qd + (uint64_t)(k * 2), kcd + (uint64_t)(k * 2), idesc_s, k != 0);
          }
          umma_commit(s_full(w));
          if (g > 0) issue_pv(g - 1, prev_kb, prev_last);
          prev_kb = kb; prev_last = (ti == nt - 1);
        }
      }
      if (G > 0) issue_pv(G - 1, prev_kb, prev_last);
    }
  } else if (warp == 10) {
    // ---------------- store warp: staged output rows -> global memory, then the stage goes back to the producer --------
    if (lane == 0) {
      for (int g = 0; g < G; ++g) {
        const int li = g / nt, ti = g - li * nt, st = g % PP_NQ, w = g & 1;
        const int it = (int)blockIdx.x + li * (int)gridDim.x;
        const int b = it / a.Hq, h = it % a.Hq;
        mbar_wait(o_staged(w), (uint32_t)((g >> 1) & 1), verr);
        if (ti < n_htiles) tma_store_3d(&maps.oh, sQ + 3 * st * SLAB, h * DH, ti * QT, b);
        else tma_store_3d(&maps.oc, sQ + 3 * st * SLAB, h * DH, (ti - n_htiles) * QT, b);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        mbar_arrive(q_free(st));
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else {
    // ---------------- softmax / epilogue: warpgroup w takes the tiles g = w, w + 2, ... ----------------
    const int w = (warp - 2) >> 2;
    const int quad = warp & 3;                       // the tensor-memory lane quarter this warp may read
    const int r = quad * 32 + lane;
    const int sw = r & 7;
    const uint32_t lane_base = ((uint32_t)(quad * 32) << 16);
    const float csc = CAP ? 1.0f : a.sm_scale * 1.4426950408889634f;
    auto wg_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + w) : "memory"); };

    // what a thread needs to know about its row of a tile; the two segment words are loaded a tile ahead of their use.
    // (li, ti) = item and tile inside the item, advanced two tiles at a time (no division per tile)
    struct Tile { int li, ti, seg, hseg; bool cand; };
    auto tile_at = [&](int li, int ti) {
      Tile t;
      t.li = li; t.ti = ti;
      const int it = (int)blockIdx.x + li * (int)gridDim.x;
      const int b = it / a.Hq;
      t.cand = ti >= n_htiles;
      const int p = (t.cand ? (ti - n_htiles) : ti) * QT + r;                        // position inside the block
      const bool in = p < (t.cand ? a.n_cand : a.n_hist);
      const long long tok = t.cand ? a.cand_row0 + (long long)b * a.cand_req_rows + p : a.hist_row0 + (long long)b * a.hist_req_rows + p;
      t.seg = in ? a.seg[tok] : 0;
      t.hseg = (r < a.n_hist) ? a.seg[a.hist_row0 + (long long)b * a.hist_req_rows + r] : 0;   // history key r of the item
      return t;
    };
    auto tile_after = [&](const Tile& c) {         // two tiles further on
      int li = c.li, ti = c.ti + 2;
      while (ti >= nt) { ti -= nt; ++li; }
      return tile_at(li, ti);
    };

    uint32_t kmask[4] = {0u, 0u, 0u, 0u};
    bool all_ok = false;
    int mask_li = -1;
    Tile cur, nxt;
    if (w < G) cur = tile_at(w / nt, w % nt);
    for (int g = w; g < G; g += 2) {
      const uint32_t ph = (uint32_t)((g >> 1) & 1);
      const int st = g % PP_NQ;
      const uint32_t stage = sQ + 3 * st * SLAB;
      const bool more = g + 2 < G;
      if (more) nxt = tile_after(cur);
      if (cur.li != mask_li) {
        // validity of the item's history keys (the same for all of its tiles)
        const uint32_t word = __ballot_sync(0xffffffffu, cur.hseg == 1);
        wg_sync();                                   // the words of the previous item have been read by every thread
        if (lane == 0) mask_words[w * 4 + quad] = word;
        wg_sync();
#pragma unroll
        for (int i = 0; i < 4; ++i) kmask[i] = mask_words[w * 4 + i];
        all_ok = (kmask[0] & kmask[1] & kmask[2] & kmask[3]) == 0xffffffffu;
        mask_li = cur.li;
      }

      mbar_wait(s_full(w), ph, verr);
      tc_fence_after();
      const bool is_cand = cur.cand && cur.seg == -1;
      // the row's score against its own key: element r of row r of the scratch (this warp's 32 x 32 diagonal block)
      float self_logit = 0.f;
      if (cur.cand) {                                // uniform over the tile
        float dv[32];
        tmem_ld32(tmem + TM_D + lane_base + quad * 32, reinterpret_cast<uint32_t*>(dv));
        tc_fence_before();
        mbar_arrive(d_free);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) dot = (lane == i) ? dv[i] : dot;
        self_logit = CAP ? capped_log2(dot, a.sm_scale, a.cap, a.cap_method) : dot * csc;
      }
      // The 128-key S row in four chunks of 32 columns, two register buffers: the load of the next chunk is in flight
      // while the current one is worked on.  Two passes (row maximum, then probabilities), each a rolled loop over
      // two pairs of chunks so that the code of a pass stays small.
      const uint32_t s_base = tmem + TM_S + w * 128 + lane_base;
      float sa[32], sb[32];
      auto fix = [&](float (&sv)[32], int c) {       // logit cap and key validity of chunk c
        if (CAP) {
#pragma unroll
          for (int k = 0; k < 32; ++k) sv[k] = capped_log2(sv[k], a.sm_scale, a.cap, a.cap_method);
        }
        if (!all_ok) {
          const uint32_t km = c == 0 ? kmask[0] : c == 1 ? kmask[1] : c == 2 ? kmask[2] : kmask[3];
#pragma unroll
          for (int k = 0; k < 32; ++k)
            if (!((km >> k) & 1u)) sv[k] = -INFINITY;
        }
      };
      auto chunk_max = [&](const float (&sv)[32]) {
        float b4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
        for (int k = 4; k + 7 < 32; k += 8) {
          b4[0] = max3f(b4[0], sv[k], sv[k + 1]); b4[1] = max3f(b4[1], sv[k + 2], sv[k + 3]);
          b4[2] = max3f(b4[2], sv[k + 4], sv[k + 5]); b4[3] = max3f(b4[3], sv[k + 6], sv[k + 7]);
        }
        b4[0] = max3f(b4[0], sv[28], sv[29]); b4[1] = max3f(b4[1], sv[30], sv[31]);
        return fmaxf(max3f(b4[0], b4[1], b4[2]), b4[3]);
      };
      // pass 1: the row maximum
      float bm = -INFINITY;
      tmem_ld32_nowait(s_base, reinterpret_cast<uint32_t*>(sa));
      tmem_ld_wait_on(sa);
#pragma unroll 1
      for (int cp = 0; cp < 2; ++cp) {
        tmem_ld32_nowait(s_base + (2 * cp + 1) * 32, reinterpret_cast<uint32_t*>(sb));
        fix(sa, 2 * cp);
        bm = fmaxf(bm, chunk_max(sa));
        tmem_ld_wait_on(sb);
        if (cp == 0) tmem_ld32_nowait(s_base + 64, reinterpret_cast<uint32_t*>(sa));
        fix(sb, 2 * cp + 1);
        bm = fmaxf(bm, chunk_max(sb));
        if (cp == 0) tmem_ld_wait_on(sa);
      }
      float m = bm * csc;
      if (is_cand) m = fmaxf(m, self_logit);           // the self key takes part in the row maximum right away
      const float mns = (m == -INFINITY) ? 0.f : m;
      // pass 2: probabilities, row sum, P as bf16 pairs back into tensor memory: chunk c of the row (32 keys) lands in
      // the 16 columns c * 16.. of the row's own S block - columns whose S values this thread has already in registers
      // or consumed (the chunk in flight lies further right)
      float l = 0.f;
      const float2 c2 = make_float2(csc, csc), n2 = make_float2(-mns, -mns);
      auto exp_chunk = [&](float (&sv)[32], int c) {
        float2 acc2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        uint32_t pw[16];
#pragma unroll
        for (int k = 0; k < 32; k += 2) {            // packed fp32: two keys per instruction; masked keys: 2^-inf = 0
          const float2 e = __ffma2_rn(make_float2(sv[k], sv[k + 1]), c2, n2);
          const float e0 = ex2f(e.x), e1 = ex2f(e.y);
          acc2[(k >> 1) & 1] = __fadd2_rn(acc2[(k >> 1) & 1], make_float2(e0, e1));
          pw[k >> 1] = pack_bf2(e0, e1);
        }
        l += (acc2[0].x + acc2[0].y) + (acc2[1].x + acc2[1].y);
        tmem_st16_nowait(s_base + c * 16, pw);
      };
      tmem_ld32_nowait(s_base, reinterpret_cast<uint32_t*>(sa));
      tmem_ld_wait_on(sa);
#pragma unroll 1
      for (int cp = 0; cp < 2; ++cp) {
        tmem_ld32_nowait(s_base + (2 * cp + 1) * 32, reinterpret_cast<uint32_t*>(sb));
        fix(sa, 2 * cp);
        exp_chunk(sa, 2 * cp);
        tmem_ld_wait_on(sb);
        if (cp == 0) tmem_ld32_nowait(s_base + 64, reinterpret_cast<uint32_t*>(sa));
        fix(sb, 2 * cp + 1);
        exp_chunk(sb, 2 * cp + 1);
        if (cp == 0) tmem_ld_wait_on(sa);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      mbar_arrive(p_ready(w));

      // while the P V product runs: the row's own value row out of the stage (128-byte swizzle: chunk c of row r sits
      // at chunk c ^ (r & 7))
      uint4 vrow[DH / 8];
      float p_self = 0.f;
      if (is_cand) {
        mbar_wait(q_full(st), (uint32_t)((g / PP_NQ) & 1), verr);   // long complete (S came from this stage): orders the reads below behind the bulk copies
#pragma unroll
        for (int c = 0; c < DH / 8; ++c)
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(vrow[c].x), "=r"(vrow[c].y), "=r"(vrow[c].z), "=r"(vrow[c].w)
                       : "r"(stage + 2 * SLAB + r * 128 + ((uint32_t)(c ^ sw) << 4)));
        p_self = ex2f(self_logit - mns);
        l += p_self;
      }
      const float pr = round_bf(p_self);
      mbar_wait(o_done(w), ph, verr);
      tc_fence_after();
      float o[DH];
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) tmem_ld32_nowait(tmem + TM_O + w * DH + lane_base + c * 32, reinterpret_cast<uint32_t*>(o) + c * 32);
      tmem_ld_wait();
      tc_fence_before();
      const float inv = (l == 0.f || cur.seg == 0) ? 0.f : 1.0f / l;   // padded rows, rows with no allowed key -> zeros
      // the output row goes into the stage's Q slab (same swizzle), from where the store warp sends the tile out; rows
      // past the end of the block are clipped by the copy
#pragma unroll
      for (int c = 0; c < DH / 8; ++c) {
        if (is_cand) {
          const float2 v0 = unpack_bf2(vrow[c].x), v1 = unpack_bf2(vrow[c].y), v2 = unpack_bf2(vrow[c].z), v3 = unpack_bf2(vrow[c].w);
          o[c * 8 + 0] += pr * v0.x; o[c * 8 + 1] += pr * v0.y; o[c * 8 + 2] += pr * v1.x; o[c * 8 + 3] += pr * v1.y;
          o[c * 8 + 4] += pr * v2.x; o[c * 8 + 5] += pr * v2.y; o[c * 8 + 6] += pr * v3.x; o[c * 8 + 7] += pr * v3.y;
        }
        uint4 ov;
        ov.x = pack_bf2(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv); ov.y = pack_bf2(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
        ov.z = pack_bf2(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv); ov.w = pack_bf2(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
        st_shared_16(stage + r * 128 + ((uint32_t)(c ^ sw) << 4), ov);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(o_staged(w));
      if (more) cur = nxt;
    }
  }

  if (*verr != 0) __nanosleep(1000000);   // error path: let in-flight bulk copies land before the CTA retires
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// tensor maps are cached: the engine calls with the same buffers every layer and every step
typedef std::tuple<const void*, long long, int, int, long long, int> MapKey;
std::map<MapKey, CUtensorMap> g_map_cache;
std::mutex g_map_mu;

phx_status cached_map3d(const CUtensorMap** out, const bf16* ptr, long long cols, int T, int B, long long tok_stride,
                        int box_rows, std::string& err) {
  std::lock_guard<std::mutex> lk(g_map_mu);
  MapKey key(ptr, cols, T, B, tok_stride, box_rows);
  auto it = g_map_cache.find(key);
  if (it == g_map_cache.end()) {
    if (g_map_cache.size() > 4096) g_map_cache.clear();
    CUtensorMap m;
    phx_status s = make_map3d(&m, ptr, cols, T, B, tok_stride * 2, (long long)T * tok_stride * 2, box_rows, err);
    if (s) return s;
    it = g_map_cache.emplace(key, m).first;
  }
  *out = &it->second;
  return PHX_OK;
}

template <bool CAP>
phx_status launch_pingpong(const AttnArgs& a, int* err_flag, int num_sms, cudaStream_t stream, std::string& err) {
  const size_t smem = (size_t)(4 + 3 * PP_NQ) * SLAB + 64 + 192 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    PHX_CUDA_TRY(cudaFuncSetAttribute(ranker_attention_pingpong_kernel<CAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), err);
    attr_set = true;
  }
  const int n_hist = a.hist_len < a.T ? a.hist_len : a.T;
  const int n_cand = a.T - n_hist;
  PingArgs p;
  p.seg = a.seg;
  p.q_head_stride = a.q_head_stride; p.k_head_stride = a.k_head_stride; p.v_head_stride = a.v_head_stride;
  p.Hq = a.Hq; p.Hkv = a.Hkv; p.n_hist = n_hist; p.n_cand = n_cand; p.n_items = a.B * a.Hq;
  p.hist_row0 = token_row(a.split, a.B, a.hist_len, a.T, 0, 0);
  p.hist_req_rows = a.split ? a.hist_len : a.T;
  p.cand_row0 = n_cand > 0 ? token_row(a.split, a.B, a.hist_len, a.T, 0, n_hist) : 0;
  p.cand_req_rows = a.split ? (a.T - a.hist_len) : a.T;
  p.skip_hist = a.q_start > 0 ? 1 : 0;
  p.sm_scale = a.sm_scale; p.cap = a.cap; p.cap_method = a.cap_method; p.err_flag = err_flag;
  if (p.skip_hist && n_cand == 0) return PHX_OK;
  // eight maps per launch: the engine calls with the same buffers every layer and every step, so they are cached whole
  struct Key {
    const void *q, *k, *v, *o; long long qs, ks, vs, h0, hr, c0, cr; int qh, kh, vh, Hq, Hkv, nh, nc, B;
    bool operator<(const Key& x) const {
      return std::tie(q, k, v, o, qs, ks, vs, h0, hr, c0, cr, qh, kh, vh, Hq, Hkv, nh, nc, B) <
             std::tie(x.q, x.k, x.v, x.o, x.qs, x.ks, x.vs, x.h0, x.hr, x.c0, x.cr, x.qh, x.kh, x.vh, x.Hq, x.Hkv, x.nh, x.nc, x.B);
    }
  };
  static std::map<Key, PingMaps> cache;
  static std::mutex mu;
  const Key key{a.q, a.k, a.v, a.out, a.q_tok_stride, a.k_tok_stride, a.v_tok_stride, p.hist_row0, p.hist_req_rows, p.cand_row0,
                p.cand_req_rows, a.q_head_stride, a.k_head_stride, a.v_head_stride, a.Hq, a.Hkv, n_hist, n_cand, a.B};
  PingMaps pm;
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
      if (cache.size() > 1024) cache.clear();
      PingMaps m;
      phx_status s;
      const long long qcols = (long long)(a.Hq - 1) * a.q_head_stride + 64, kcols = (long long)(a.Hkv - 1) * a.k_head_stride + 64,
                      vcols = (long long)(a.Hkv - 1) * a.v_head_stride + 64, ocols = (long long)a.Hq * 64;
      const long long ostr = ocols;   // output rows are dense: [token][head][64]
      auto mk = [&](CUtensorMap* dst, const bf16* ptr, long long cols, long long rows, long long tok_stride, long long req_rows) {
        return sm100::make_map3d(dst, ptr, cols, rows, a.B, tok_stride * 2, req_rows * tok_stride * 2, 128, err);
      };
      if ((s = mk(&m.qh, a.q + p.hist_row0 * a.q_tok_stride, qcols, n_hist, a.q_tok_stride, p.hist_req_rows))) return s;
      if ((s = mk(&m.kh, a.k + p.hist_row0 * a.k_tok_stride, kcols, n_hist, a.k_tok_stride, p.hist_req_rows))) return s;
      if ((s = mk(&m.vh, a.v + p.hist_row0 * a.v_tok_stride, vcols, n_hist, a.v_tok_stride, p.hist_req_rows))) return s;
      if ((s = mk(&m.oh, a.out + p.hist_row0 * ostr, ocols, n_hist, ostr, p.hist_req_rows))) return s;
      m.qc = m.qh; m.kc = m.kh; m.vc = m.vh; m.oc = m.oh;
      if (n_cand > 0) {
        if ((s = mk(&m.qc, a.q + p.cand_row0 * a.q_tok_stride, qcols, n_cand, a.q_tok_stride, p.cand_req_rows))) return s;
        if ((s = mk(&m.kc, a.k + p.cand_row0 * a.k_tok_stride, kcols, n_cand, a.k_tok_stride, p.cand_req_rows))) return s;
        if ((s = mk(&m.vc, a.v + p.cand_row0 * a.v_tok_stride, vcols, n_cand, a.v_tok_stride, p.cand_req_rows))) return s;
        if ((s = mk(&m.oc, a.out + p.cand_row0 * ostr, ocols, n_cand, ostr, p.cand_req_rows))) return s;
      }
      it = cache.emplace(key, m).first;
    }
    pm = it->second;
  }
  const int grid = p.n_items < num_sms ? p.n_items : num_sms;
  ranker_attention_pingpong_kernel<CAP><<<grid, PP_THREADS, smem, stream>>>(pm, p);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

template <int DH, bool CAP>
phx_status launch_tc(const AttnArgs& a, int* err_flag, cudaStream_t stream, std::string& err) {
  constexpr int KBLK = (DH == 64) ? 128 : 64;
  constexpr int DCH = DH / 64;
  constexpr int NSB = (KBLK <= 64) ? 2 : 1;   // K buffers, as in the kernel
  const size_t smem = (size_t)DCH * SLAB + (NSB + 2) * (size_t)DCH * KBLK * 128 + TC_MAX_BLOCKS * 16 + 128 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    PHX_CUDA_TRY(cudaFuncSetAttribute(ranker_attention_tc_kernel<DH, CAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), err);
    attr_set = true;
  }
  const CUtensorMap *mq, *mk, *mv, *mo;
  phx_status s;
  if ((s = cached_map3d(&mq, a.q, (long long)(a.Hq - 1) * a.q_head_stride + DH, a.T, a.B, a.q_tok_stride, QT, err))) return s;
  if ((s = cached_map3d(&mk, a.k, (long long)(a.Hkv - 1) * a.k_head_stride + DH, a.T, a.B, a.k_tok_stride, KBLK, err))) return s;
  if ((s = cached_map3d(&mv, a.v, (long long)(a.Hkv - 1) * a.v_head_stride + DH, a.T, a.B, a.v_tok_stride, KBLK, err))) return s;
  if ((s = cached_map3d(&mo, a.out, (long long)a.Hq * DH, a.T, a.B, (long long)a.Hq * DH, QT, err))) return s;
  AttnTcArgs t;
  t.q = a.q; t.k = a.k; t.v = a.v; t.out = a.out;
  t.q_tok_stride = a.q_tok_stride; t.k_tok_stride = a.k_tok_stride; t.v_tok_stride = a.v_tok_stride;
  t.q_head_stride = a.q_head_stride; t.k_head_stride = a.k_head_stride; t.v_head_stride = a.v_head_stride;
  t.seg = a.seg; t.B = a.B; t.T = a.T; t.Hq = a.Hq; t.Hkv = a.Hkv; t.hist_len = a.hist_len;
  t.sm_scale = a.sm_scale; t.cap = a.cap; t.cap_method = a.cap_method; t.err_flag = err_flag;
  dim3 grid((a.T + QT - 1) / QT, a.Hq, a.B);
  ranker_attention_tc_kernel<DH, CAP><<<grid, A_THREADS, smem, stream>>>(*mq, *mk, *mv, *mo, t);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status launch_resident(const AttnArgs& a, int* err_flag, cudaStream_t stream, std::string& err) {
  const size_t smem = 6 * (size_t)SLAB + 64 + 128 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    PHX_CUDA_TRY(cudaFuncSetAttribute(ranker_attention_resident_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), err);
    attr_set = true;
  }
  const CUtensorMap *mq, *mk, *mv, *mo;
  phx_status s;
  if ((s = cached_map3d(&mq, a.q, (long long)(a.Hq - 1) * a.q_head_stride + 64, a.T, a.B, a.q_tok_stride, QT, err))) return s;
  if ((s = cached_map3d(&mk, a.k, (long long)(a.Hkv - 1) * a.k_head_stride + 64, a.T, a.B, a.k_tok_stride, 128, err))) return s;
  if ((s = cached_map3d(&mv, a.v, (long long)(a.Hkv - 1) * a.v_head_stride + 64, a.T, a.B, a.v_tok_stride, 128, err))) return s;
  if ((s = cached_map3d(&mo, a.out, (long long)a.Hq * 64, a.T, a.B, (long long)a.Hq * 64, QT, err))) return s;
  AttnTcArgs t;
  t.q = a.q; t.k = a.k; t.v = a.v; t.out = a.out;
  t.q_tok_stride = a.q_tok_stride; t.k_tok_stride = a.k_tok_stride; t.v_tok_stride = a.v_tok_stride;
  t.q_head_stride = a.q_head_stride; t.k_head_stride = a.k_head_stride; t.v_head_stride = a.v_head_stride;
  t.seg = a.seg; t.B = a.B; t.T = a.T; t.Hq = a.Hq; t.Hkv = a.Hkv; t.hist_len = a.hist_len;
  t.sm_scale = a.sm_scale; t.cap = a.cap; t.cap_method = a.cap_method; t.err_flag = err_flag;
  const int cap_on = (a.cap_method != 0 && a.cap > 0.f) ? 1 : 0;
  dim3 grid(1, a.Hq, a.B);
  ranker_attention_resident_kernel<<<grid, A_THREADS, smem, stream>>>(*mq, *mk, *mv, *mo, t, cap_on);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

}  // namespace

// the two-warpgroup resident-history kernel: head dim 64, 1..128 history keys, q heads not grouped, rows not packed
bool ranker_attention_pingpong_supported(const AttnArgs& a) {
  const int n_hist = a.hist_len < a.T ? a.hist_len : a.T;
  if (a.dh != 64 || n_hist < 1 || n_hist > 128 || a.q_group > 1 || a.pack.hist_off || a.Hq % a.Hkv != 0) return false;
  if (a.q_start != 0 && a.q_start != n_hist) return false;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return al(a.q) && al(a.k) && al(a.v) && al(a.out) && a.q_tok_stride % 8 == 0 && a.k_tok_stride % 8 == 0 &&
         a.v_tok_stride % 8 == 0 && a.q_head_stride % 8 == 0 && a.k_head_stride % 8 == 0 && a.v_head_stride % 8 == 0;
}

phx_status ranker_attention_pingpong_launch(const AttnArgs& a, int* err_flag, cudaStream_t stream, std::string& err) {
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  dispatch_note(DK_ATTN_PINGPONG);
  const bool cap = a.cap_method != 0 && a.cap > 0.f;
  return cap ? launch_pingpong<true>(a, err_flag, num_sms, stream, err) : launch_pingpong<false>(a, err_flag, num_sms, stream, err);
}

bool ranker_attention_tc_supported(const AttnArgs& a) {
  if (a.dh != 64 && a.dh != 128) return false;
  if (a.q_group > 1) return false;   // grouped q heads of a merged QKV row: the mma.sync kernels address them
  {
    const int n_hist = a.hist_len < a.T ? a.hist_len : a.T;
    if ((n_hist + 63) / 64 > TC_MAX_BLOCKS) return false;   // validity table of the CTA
  }
  // TMA: 16-byte aligned bases and strides, head offsets that are multiples of 8 elements
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return al(a.q) && al(a.k) && al(a.v) && al(a.out) && a.q_tok_stride % 8 == 0 && a.k_tok_stride % 8 == 0 &&
         a.v_tok_stride % 8 == 0 && a.q_head_stride % 8 == 0 && a.k_head_stride % 8 == 0 && a.v_head_stride % 8 == 0;
}

phx_status ranker_attention_tc_launch(const AttnArgs& a, int* err_flag, cudaStream_t stream, std::string& err) {
  const bool cap = a.cap_method != 0 && a.cap > 0.f;
  {
    const char* force = getenv("PHX_ATTN");
    const bool resident = force && strcmp(force, "resident") == 0;
    const int n_hist = a.hist_len < a.T ? a.hist_len : a.T;
    if (resident && a.dh == 64 && n_hist <= 128 && n_hist > 0) { dispatch_note(DK_ATTN_RESIDENT); return launch_resident(a, err_flag, stream, err); }
  }
  dispatch_note(DK_ATTN_TC);
  if (a.dh == 64) return cap ? launch_tc<64, true>(a, err_flag, stream, err) : launch_tc<64, false>(a, err_flag, stream, err);
  if (a.dh == 128) return cap ? launch_tc<128, true>(a, err_flag, stream, err) : launch_tc<128, false>(a, err_flag, stream, err);
  err = "attention (tcgen05): head dim must be 64 or 128";
  return PHX_E_ARG;
}

}  // namespace phx
