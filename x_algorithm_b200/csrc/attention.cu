// Candidate-isolated ("ranker") attention: every valid query attends to the valid history keys, a
// candidate additionally to itself and to no other candidate, padded queries produce zeros
// (mask: phoenix/xrex/pallas/ranker_attention_utils.py:16-56; kernel form
// phoenix/xrex/pallas/ranker_attention_v2.py:113-148, 183).
//
// The candidate x candidate block is never formed: only the history keys stream through shared memory
// (64 keys per step, two cp.async buffers) and a candidate's single self key is folded in as one extra
// online-softmax step computed as a per-row dot product.  One CTA = 128 query rows of one
// (batch, head): 8 warps x 16 rows.  Everything a CTA needs at the start (Q tile, the tile's own K/V rows
// for the self term, the first two key blocks) is requested up front with cp.async, so a history of
// <= 128 keys costs a single round trip to L2/HBM.  S = Q K^T and O += P V run on mma.sync m16n8k16
// bf16 with fp32 accumulation, fragments come from padded shared memory through ldmatrix, P is rounded
// to bf16 before P V as the reference does, and the output tile is staged in shared memory so global
// stores are full 16-byte chunks of contiguous rows.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace phx {
namespace {

constexpr int KB = 64;           // keys per step
constexpr int ATT_WARPS = 8;
constexpr int QROWS = 16 * ATT_WARPS;
constexpr int ATT_THREADS = 32 * ATT_WARPS;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src, bool pred) {
  const int sz = pred ? 16 : 0;  // size 0 -> the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// logits are kept in the log2 domain: value = cap(s * sm_scale) * log2(e)
__device__ __forceinline__ float scaled_logit(float s, float sm_scale, float cap, int method) {
  const float LOG2E = 1.4426950408889634f;
  float v = s * sm_scale;
  if (method == 1) v = v / (1.0f + fabsf(v) / cap);   // soft_sign
  else if (method == 2) v = cap * tanhf(v / cap);     // tanh
  return v * LOG2E;
}

// CAP = false: logits stay raw accumulators and the scale sm_scale * log2(e) is folded into the exponent's FMA
template <int DH, bool CAP>
__global__ void __launch_bounds__(ATT_THREADS) ranker_attention_kernel(AttnArgs a) {
  constexpr int LD = DH + 8;          // padded row (elements): conflict-free ldmatrix
  constexpr int KSTEPS = DH / 16;     // k-steps of Q K^T
  constexpr int DT = DH / 8;          // output n-tiles
  constexpr int CH = DH / 8;          // 16-byte chunks per row
  extern __shared__ __align__(128) uint8_t asm_raw[];
  bf16* sq = reinterpret_cast<bf16*>(asm_raw);     // [QROWS][LD]  Q tile, later the output tile
  bf16* sks = sq + QROWS * LD;                     // [QROWS][LD]  K rows of the tile's own tokens
  bf16* svs = sks + QROWS * LD;                    // [QROWS][LD]  V rows of the tile's own tokens
  bf16* skv = svs + QROWS * LD;                    // [2][2][KB][LD]  key-block ring: (buffer, K|V)
  int* skey_ok = reinterpret_cast<int*>(skv + 4 * KB * LD);  // [2][KB]
  int* sall_ok = skey_ok + 2 * KB;                           // [2][2] per buffer and 32-key half: all keys valid history
  const float csc = CAP ? 1.0f : a.sm_scale * 1.4426950408889634f;
  // programmatic dependent launch: the kernel may have been started before the one in front of it on the stream
  // finished; wait for that one before reading what it wrote, and let the kernel behind begin its own set-up
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * QROWS;
  // rows of this request: the batch's common shape, or its own counts when the rows are packed
  int T = a.T, hist_len = a.hist_len, q_start = a.q_start;
  if (a.pack.on()) {
    hist_len = a.pack.hist_cnt(b);
    T = hist_len + a.pack.cand_cnt(b);
    if (q_start > 0) q_start = hist_len;
  }
  if (q0 >= T || q0 + QROWS <= q_start) return;   // past the request's rows, or history queries of a candidate-only layer
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  // token row of position t of this request: in every layout (plain, split, packed) the history slots are one run of
  // consecutive rows and the candidate slots another
  const int n_hist = hist_len < T ? hist_len : T;
  int hrow0, crow0;   // row of t = hrow0 + t in front of n_hist, crow0 + t from there on (token rows fit 31 bits)
  if (a.pack.on()) { hrow0 = a.pack.hist_off[b]; crow0 = (int)(a.pack.cand_base + a.pack.cand_off[b]) - n_hist; }
  else { hrow0 = (int)token_row(a.split, a.B, hist_len, T, b, 0); crow0 = (int)token_row(a.split, a.B, hist_len, T, b, n_hist) - n_hist; }
  auto trow = [&](int t) -> long long { return (long long)((t < n_hist ? hrow0 : crow0) + t); };
  const int n_blocks = (n_hist + KB - 1) / KB;
  const bool has_cand = (q0 + QROWS > n_hist);     // rows at or past hist_len may be candidates

  const bf16* kbase = a.k + (long long)hk * a.k_head_stride;
  const bf16* vbase = a.v + (long long)hk * a.v_head_stride;

  auto load_block = [&](int blk, int buf) {
    bf16* dk = skv + (size_t)(buf * 2 + 0) * KB * LD;
    bf16* dv = skv + (size_t)(buf * 2 + 1) * KB * LD;
    for (int c = threadIdx.x; c < KB * CH; c += ATT_THREADS) {
      const int kr = c / CH, dc = (c % CH) * 8;
      const int key = blk * KB + kr;
      const bool ok = key < n_hist;
      const long long tok = trow(ok ? key : 0);
      cp16((uint32_t)__cvta_generic_to_shared(dk + kr * LD + dc), kbase + tok * a.k_tok_stride + dc, ok);
      cp16((uint32_t)__cvta_generic_to_shared(dv + kr * LD + dc), vbase + tok * a.v_tok_stride + dc, ok);
    }
    if (threadIdx.x < KB) {  // warps 0 and 1
      const int key = blk * KB + threadIdx.x;
      const int ok = (key < n_hist) && (a.seg[trow(key)] == 1);
      skey_ok[buf * KB + threadIdx.x] = ok;
      const int all32 = __all_sync(0xffffffffu, ok);
      if ((threadIdx.x & 31) == 0) sall_ok[buf * 2 + (threadIdx.x >> 5)] = all32;
    }
  };

  // ---- prologue: Q tile, own K/V rows, key blocks 0 and 1 --------------------------------------------
  for (int c = threadIdx.x; c < QROWS * CH; c += ATT_THREADS) {
    const int r = c / CH, dc = (c % CH) * 8;
    const bool ok = (q0 + r) < T;
    const long long tok = trow(ok ? q0 + r : 0);
    cp16((uint32_t)__cvta_generic_to_shared(sq + r * LD + dc), a.q + tok * a.q_tok_stride + a.q_col(h) + dc, ok);
    if (has_cand) {
      cp16((uint32_t)__cvta_generic_to_shared(sks + r * LD + dc), kbase + tok * a.k_tok_stride + dc, ok);
      cp16((uint32_t)__cvta_generic_to_shared(svs + r * LD + dc), vbase + tok * a.v_tok_stride + dc, ok);
    }
  }
  if (n_blocks > 0) load_block(0, 0);
  cp_commit();
  if (n_blocks > 1) load_block(1, 1);
  cp_commit();

  const int rq[2] = {q0 + warp * 16 + g, q0 + warp * 16 + g + 8};
  int segq[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) segq[i] = (rq[i] < T) ? a.seg[trow(rq[i])] : 0;

  cp_wait<1>();
  __syncthreads();

  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
            (uint32_t)__cvta_generic_to_shared(sq + (warp * 16 + (lane & 15)) * LD + ks * 16 + ((lane >> 4) << 3)));

  float o[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m[2] = {-INFINITY, -INFINITY}, mprev[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int blk = 0; blk < n_blocks; ++blk) {
    const int buf = blk & 1;
    if (blk > 0) {
      if (blk + 1 < n_blocks) cp_wait<1>(); else cp_wait<0>();
      __syncthreads();
    }
    const bf16* sk = skv + (size_t)(buf * 2 + 0) * KB * LD;
    const bf16* sv = skv + (size_t)(buf * 2 + 1) * KB * LD;
    const int* kok = skey_ok + buf * KB;

    // S = Q K^T for 64 keys: 8 n-tiles of 8 keys, two per ldmatrix.x4
    float s[KB / 8][4];
#pragma unroll
    for (int j = 0; j < KB / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {       // k-step outermost: the 8 accumulator chains stay independent
#pragma unroll
      for (int j = 0; j < KB / 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        // lanes 0-7: keys j*8.., d ks*16; 8-15: same keys, d +8; 16-23: keys (j+1)*8.., d ks*16; 24-31: d +8
        const int kr = j * 8 + (lane & 7) + ((lane >> 4) << 3);
        const int kc = ks * 16 + (((lane >> 3) & 1) << 3);
        ldsm_x4(b0, b1, b2, b3, (uint32_t)__cvta_generic_to_shared(sk + kr * LD + kc));
        mma_bf16_16816(s[j], qf[ks], b0, b1);
        mma_bf16_16816(s[j + 1], qf[ks], b2, b3);
      }
    }
    // (cap,) key mask only where the block holds invalid keys, block max.  Padded query rows are not masked
    // here: their output is forced to zero at the end.
    if (CAP) {
#pragma unroll
      for (int j = 0; j < KB / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = scaled_logit(s[j][e], a.sm_scale, a.cap, a.cap_method);
    }
    if (!(sall_ok[buf * 2] & sall_ok[buf * 2 + 1])) {
#pragma unroll
      for (int j = 0; j < KB / 8; ++j) {
        const int2 okp = *reinterpret_cast<const int2*>(&kok[j * 8 + 2 * t4]);
        if (!okp.x) { s[j][0] = -INFINITY; s[j][2] = -INFINITY; }
        if (!okp.y) { s[j][1] = -INFINITY; s[j][3] = -INFINITY; }
      }
    }
    float bm[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < KB / 8; ++j) {
      bm[0] = fmaxf(bm[0], fmaxf(s[j][0], s[j][1]));
      bm[1] = fmaxf(bm[1], fmaxf(s[j][2], s[j][3]));
    }
    float alpha[2], mn[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      bm[i] = fmaxf(bm[i], __shfl_xor_sync(0xffffffffu, bm[i], 1));
      bm[i] = fmaxf(bm[i], __shfl_xor_sync(0xffffffffu, bm[i], 2));
      m[i] = fmaxf(m[i], bm[i] * csc);                 // running max, log2 domain
      mn[i] = (m[i] == -INFINITY) ? 0.f : m[i];        // finite stand-in while nothing is allowed yet
      alpha[i] = ex2(mprev[i] - mn[i]);                // -inf - finite -> 0
      mprev[i] = m[i];
    }
    // P = 2^(S - m); row sums of the unrounded p in fp32; P rounded to bf16 for P V
    uint32_t pf[KB / 16][4];
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < KB / 8; ++j) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ri = e >> 1;
        p[e] = ex2(fmaf(s[j][e], csc, -mn[ri]));      // masked logit: -inf -> 0
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
        ldsm_x4_trans(b0, b1, b2, b3,
                      (uint32_t)__cvta_generic_to_shared(sv + (kk * 16 + (lane & 15)) * LD + jd * 8 + ((lane >> 4) << 3)));
        mma_bf16_16816(o[jd], pf[kk], b0, b1);
        mma_bf16_16816(o[jd + 1], pf[kk], b2, b3);
      }
    }
    // refill this buffer with block blk+2
    if (blk + 2 < n_blocks) {
      __syncthreads();
      load_block(blk + 2, buf);
      cp_commit();
    }
  }

  // ---- self key of candidate rows: one more online-softmax step with a per-row dot product ------------
  if (has_cand) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const bool is_cand = segq[i] == -1;
      const int lr = warp * 16 + g + 8 * i;  // row inside the tile
      float dot = 0.f;
      if (is_cand) {
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          const float2 qa = unpack_bf2(qf[ks][i]), qb = unpack_bf2(qf[ks][i + 2]);
          const float2 ka = unpack_bf2(*reinterpret_cast<const uint32_t*>(sks + lr * LD + ks * 16 + 2 * t4));
          const float2 kb = unpack_bf2(*reinterpret_cast<const uint32_t*>(sks + lr * LD + ks * 16 + 2 * t4 + 8));
          dot += qa.x * ka.x + qa.y * ka.y + qb.x * kb.x + qb.y * kb.y;
        }
      }
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      if (is_cand) {
        const float sv_ = CAP ? scaled_logit(dot, a.sm_scale, a.cap, a.cap_method) : dot * csc;
        const float mn = fmaxf(m[i], sv_);
        const float alpha = ex2(m[i] - mn);             // no history yet: 2^-inf = 0
        const float p = ex2(sv_ - mn);
        const float pr = round_bf(p);
        l[i] = l[i] * alpha + p;
        m[i] = mn;
#pragma unroll
        for (int j = 0; j < DT; ++j) {
          const float2 vv = unpack_bf2(*reinterpret_cast<const uint32_t*>(svs + lr * LD + j * 8 + 2 * t4));
          o[j][2 * i + 0] = o[j][2 * i + 0] * alpha + pr * vv.x;
          o[j][2 * i + 1] = o[j][2 * i + 1] * alpha + pr * vv.y;
        }
      }
    }
  }

  // ---- normalise, stage the warp's 16 x DH output rows in the (now free) Q tile, store 16-byte chunks --
  // each warp only ever touched its own 16 rows of sq after the first barrier, so a warp-level sync suffices
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float inv = (l[i] == 0.f || segq[i] == 0) ? 0.f : 1.0f / l[i];   // padded rows, rows with no allowed key -> zeros
    bf16* orow = sq + (warp * 16 + g + 8 * i) * LD;
#pragma unroll
    for (int j = 0; j < DT; ++j)
      *reinterpret_cast<uint32_t*>(orow + j * 8 + 2 * t4) = pack_bf2(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
  }
  __syncwarp();
  for (int c = lane; c < 16 * CH; c += 32) {
    const int r = c / CH, dc = (c % CH) * 8;
    const int row = q0 + warp * 16 + r;
    if (row < T)
      *reinterpret_cast<uint4*>(a.out + (trow(row) * a.Hq + h) * DH + dc) =
          *reinterpret_cast<const uint4*>(sq + (warp * 16 + r) * LD + dc);
  }
}

// launch with the attribute that lets the kernel start while its predecessor on the stream drains (the kernels wait
// before they read global memory); PHX_PDL=0 keeps plain stream order
template <typename Kern>
cudaError_t launch_overlapped(Kern kern, dim3 grid, int threads, size_t smem, cudaStream_t stream, const AttnArgs& a) {
  cudaLaunchConfig_t lc;
  memset(&lc, 0, sizeof(lc));
  lc.gridDim = grid; lc.blockDim = dim3(threads); lc.dynamicSmemBytes = smem; lc.stream = stream;
  cudaLaunchAttribute at[1];
  static const bool pdl = !(getenv("PHX_PDL") && getenv("PHX_PDL")[0] == '0');
  if (pdl) {
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&lc, kern, a);
}

template <int DH, bool CAP>
phx_status launch_dh(const AttnArgs& a, cudaStream_t stream, std::string& err) {
  constexpr int LD = DH + 8;
  const size_t smem = (size_t)(3 * QROWS + 4 * KB) * LD * 2 + (2 * KB + 4) * sizeof(int);
  static bool attr_set = false;
  if (!attr_set) {
    PHX_CUDA_TRY(cudaFuncSetAttribute(ranker_attention_kernel<DH, CAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), err);
    attr_set = true;
  }
  dim3 grid((a.T + QROWS - 1) / QROWS, a.Hq, a.B);
  PHX_CUDA_TRY(launch_overlapped(ranker_attention_kernel<DH, CAP>, grid, ATT_THREADS, smem, stream, a), err);
  return PHX_OK;
}


// ---- resident-history variant for head dim 64 and a history of at most 128 keys --------------------------------
// One CTA = one (batch, head): the history K/V (<= 128 x 64) is loaded once and stays in shared memory while the
// CTA walks over all query tiles of the request.  Each warp owns a 16-row strip per tile and runs its own cp.async
// pipeline: the strip's Q rows for tile i+1 are requested right after tile i's Q fragments are in registers, its
// own K/V rows (for the candidates' self key) right after tile i's self term, so every load has a whole tile of
// tensor work to hide behind and, after the prologue, no CTA-wide barrier is needed.  Rows are 128 bytes with the
// 16-byte chunk index XOR-ed with (row & 7): conflict-free ldmatrix without padding, 96 KB per CTA, two CTAs per SM.
constexpr int STRIP_HIST = 128;
constexpr int STRIP_SMEM = 2 * STRIP_HIST * 64 * 2 + ATT_WARPS * 4 * 16 * 64 * 2 + (STRIP_HIST + 4) * (int)sizeof(int);

__device__ __forceinline__ int swz(int row, int chunk) { return row * 64 + ((chunk ^ (row & 7)) << 3); }   // element offset

template <bool CAP>
__global__ void __launch_bounds__(ATT_THREADS, 2) ranker_attention_strip_kernel(AttnArgs a) {
  constexpr int DH = 64, KSTEPS = 4, DT = 8, CH = 8;
  extern __shared__ __align__(128) uint8_t asm_raw[];
  bf16* hk_s = reinterpret_cast<bf16*>(asm_raw);                 // [128][64] history K
  bf16* hv_s = hk_s + STRIP_HIST * 64;                            // [128][64] history V
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  bf16* wbase = hv_s + STRIP_HIST * 64 + warp * (4 * 16 * 64);    // this warp's strip buffers
  auto wq = [&](int i) { return wbase + (i & 1) * (16 * 64); };   // Q strip (double-buffered), later the output strip
  bf16* wks = wbase + 2 * 16 * 64;                                // K rows of the strip's own tokens
  bf16* wvs = wbase + 3 * 16 * 64;                                // V rows of the strip's own tokens
  int* skey_ok = reinterpret_cast<int*>(hv_s + STRIP_HIST * 64 + ATT_WARPS * 4 * 16 * 64);   // [128]
  int* sall_ok = skey_ok + STRIP_HIST;                                                       // [4] per 32 keys
  const float csc = CAP ? 1.0f : a.sm_scale * 1.4426950408889634f;
  // programmatic dependent launch: the kernel may have been started before the one in front of it on the stream
  // finished; wait for that one before reading what it wrote, and let the kernel behind begin its own set-up
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int b = blockIdx.y, h = blockIdx.x;
  const int hk = h / (a.Hq / a.Hkv);
  const int g = lane >> 2, t4 = lane & 3;
  int T = a.T, hist_len = a.hist_len, q_start = a.q_start;   // the batch's common shape, or this request's own counts
  if (a.pack.on()) {
    hist_len = a.pack.hist_cnt(b);
    T = hist_len + a.pack.cand_cnt(b);
    if (q_start > 0) q_start = hist_len;
  }
  // token row of position t of this request: in every layout (plain, split, packed) the history slots are one run of
  // consecutive rows and the candidate slots another
  const int n_hist = hist_len < T ? hist_len : T;
  int hrow0, crow0;   // row of t = hrow0 + t in front of n_hist, crow0 + t from there on (token rows fit 31 bits)
  if (a.pack.on()) { hrow0 = a.pack.hist_off[b]; crow0 = (int)(a.pack.cand_base + a.pack.cand_off[b]) - n_hist; }
  else { hrow0 = (int)token_row(a.split, a.B, hist_len, T, b, 0); crow0 = (int)token_row(a.split, a.B, hist_len, T, b, n_hist) - n_hist; }
  auto trow = [&](int t) -> long long { return (long long)((t < n_hist ? hrow0 : crow0) + t); };
  const int n_blocks = (n_hist + KB - 1) / KB;
  const int n_tiles = (T + QROWS - 1) / QROWS;
  const bf16* qbase = a.q + a.q_col(h);
  const bf16* kbase = a.k + (long long)hk * a.k_head_stride;
  const bf16* vbase = a.v + (long long)hk * a.v_head_stride;

  auto load_q = [&](int tile, bf16* dst) {     // this warp's 16 Q rows of `tile`
    const int r0 = tile * QROWS + warp * 16;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = lane + 32 * k, r = c >> 3, ch = c & 7;
      const bool ok = (r0 + r) < T;
      const long long tok = trow(ok ? r0 + r : 0);
      cp16((uint32_t)__cvta_generic_to_shared(dst + swz(r, ch)), qbase + tok * a.q_tok_stride + ch * 8, ok);
    }
  };
  auto strip_has_cand = [&](int tile) {
    const int r0 = tile * QROWS + warp * 16;
    return r0 < T && r0 + 16 > n_hist;
  };
  auto load_own_kv = [&](int tile) {
    const int r0 = tile * QROWS + warp * 16;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = lane + 32 * k, r = c >> 3, ch = c & 7;
      const bool ok = (r0 + r) < T;
      const long long tok = trow(ok ? r0 + r : 0);
      cp16((uint32_t)__cvta_generic_to_shared(wks + swz(r, ch)), kbase + tok * a.k_tok_stride + ch * 8, ok);
      cp16((uint32_t)__cvta_generic_to_shared(wvs + swz(r, ch)), vbase + tok * a.v_tok_stride + ch * 8, ok);
    }
  };

  // ---- prologue: history K/V for the CTA, strip 0 for each warp ----------------------------------------
  for (int c = threadIdx.x; c < STRIP_HIST * CH; c += ATT_THREADS) {
    const int kr = c >> 3, ch = c & 7;
    const bool ok = kr < n_hist;
    const long long tok = trow(ok ? kr : 0);
    cp16((uint32_t)__cvta_generic_to_shared(hk_s + swz(kr, ch)), kbase + tok * a.k_tok_stride + ch * 8, ok);
    cp16((uint32_t)__cvta_generic_to_shared(hv_s + swz(kr, ch)), vbase + tok * a.v_tok_stride + ch * 8, ok);
  }
  if (threadIdx.x < STRIP_HIST) {   // warps 0..3
    const int key = threadIdx.x;
    const int ok = (key < n_hist) && (a.seg[trow(key)] == 1);
    skey_ok[key] = ok;
    const int all32 = __all_sync(0xffffffffu, ok);
    if (lane == 0) sall_ok[key >> 5] = all32;
  }
  const int tile0 = q_start / QROWS;   // candidate-only layer: query tiles in front of q_start are not wanted
  load_q(tile0, wq(tile0));
  if (strip_has_cand(tile0)) load_own_kv(tile0);
  cp_commit();
  cp_wait<0>();
  __syncthreads();

  for (int tile = tile0; tile < n_tiles; ++tile) {
    const int q0 = tile * QROWS;
    bf16* sq = wq(tile);
    const int rq[2] = {q0 + warp * 16 + g, q0 + warp * 16 + g + 8};
    int segq[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) segq[i] = (rq[i] < T) ? a.seg[trow(rq[i])] : 0;
    const bool has_cand = strip_has_cand(tile);

    if (tile > tile0) { cp_wait<1>(); __syncwarp(); }   // this tile's Q strip has landed (its own K/V may still be in flight)
    uint32_t qf[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
      ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
              (uint32_t)__cvta_generic_to_shared(sq + swz(lane & 15, ks * 2 + (lane >> 4))));
    __syncwarp();
    if (tile + 1 < n_tiles) load_q(tile + 1, wq(tile + 1));   // that buffer's last reader was tile-1's output copy
    cp_commit();

    float o[DT][4];
#pragma unroll
    for (int j = 0; j < DT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, mprev[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (q0 + warp * 16 < T) {
      for (int blk = 0; blk < n_blocks; ++blk) {
        const bf16* sk = hk_s + blk * KB * 64;     // KB is a multiple of 8: the swizzle phase is unchanged
        const bf16* sv = hv_s + blk * KB * 64;
        const int* kok = skey_ok + blk * KB;
        float s[KB / 8][4];
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
          for (int j = 0; j < KB / 8; j += 2) {
            uint32_t b0, b1, b2, b3;
            const int kr = j * 8 + (lane & 7) + ((lane >> 4) << 3);
            const int kc = ks * 2 + ((lane >> 3) & 1);
            ldsm_x4(b0, b1, b2, b3, (uint32_t)__cvta_generic_to_shared(sk + swz(kr, kc)));
            mma_bf16_16816(s[j], qf[ks], b0, b1);
            mma_bf16_16816(s[j + 1], qf[ks], b2, b3);
          }
        }
        if (CAP) {
#pragma unroll
          for (int j = 0; j < KB / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = scaled_logit(s[j][e], a.sm_scale, a.cap, a.cap_method);
        }
        if (!(sall_ok[blk * 2] & sall_ok[blk * 2 + 1])) {
#pragma unroll
          for (int j = 0; j < KB / 8; ++j) {
            const int2 okp = *reinterpret_cast<const int2*>(&kok[j * 8 + 2 * t4]);
            if (!okp.x) { s[j][0] = -INFINITY; s[j][2] = -INFINITY; }
            if (!okp.y) { s[j][1] = -INFINITY; s[j][3] = -INFINITY; }
          }
        }
        float bm[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
          bm[0] = fmaxf(bm[0], fmaxf(s[j][0], s[j][1]));
          bm[1] = fmaxf(bm[1], fmaxf(s[j][2], s[j][3]));
        }
        float alpha[2], mn[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          bm[i] = fmaxf(bm[i], __shfl_xor_sync(0xffffffffu, bm[i], 1));
          bm[i] = fmaxf(bm[i], __shfl_xor_sync(0xffffffffu, bm[i], 2));
          m[i] = fmaxf(m[i], bm[i] * csc);
          mn[i] = (m[i] == -INFINITY) ? 0.f : m[i];
          alpha[i] = ex2(mprev[i] - mn[i]);
          mprev[i] = m[i];
        }
        // P = 2^(S - m) with packed fp32 arithmetic (two columns of a row per instruction)
        uint32_t pf[KB / 16][4];
        float2 ls2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        const float2 csc2 = make_float2(csc, csc);
        const float2 nm2[2] = {make_float2(-mn[0], -mn[0]), make_float2(-mn[1], -mn[1])};
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
#pragma unroll
          for (int ri = 0; ri < 2; ++ri) {
            const float2 e = __ffma2_rn(make_float2(s[j][2 * ri], s[j][2 * ri + 1]), csc2, nm2[ri]);
            const float2 pp = make_float2(ex2(e.x), ex2(e.y));      // masked logit: -inf -> 0
            ls2[ri] = __fadd2_rn(ls2[ri], pp);
            pf[j >> 1][(j & 1) * 2 + ri] = pack_bf2(pp.x, pp.y);
          }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // a row's 64 probabilities are spread over the 4 lanes of its quad
          float lsum = ls2[i].x + ls2[i].y;
          lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
          lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
          l[i] = l[i] * alpha[i] + lsum;
        }
        if (blk > 0) {   // nothing to rescale before the first block
          const float2 a0 = make_float2(alpha[0], alpha[0]), a1 = make_float2(alpha[1], alpha[1]);
#pragma unroll
          for (int j = 0; j < DT; ++j) {
            const float2 x = __fmul2_rn(make_float2(o[j][0], o[j][1]), a0), y = __fmul2_rn(make_float2(o[j][2], o[j][3]), a1);
            o[j][0] = x.x; o[j][1] = x.y; o[j][2] = y.x; o[j][3] = y.y;
          }
        }
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
#pragma unroll
          for (int jd = 0; jd < DT; jd += 2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(b0, b1, b2, b3,
                          (uint32_t)__cvta_generic_to_shared(sv + swz(kk * 16 + (lane & 15), jd + (lane >> 4))));
            mma_bf16_16816(o[jd], pf[kk], b0, b1);
            mma_bf16_16816(o[jd + 1], pf[kk], b2, b3);
          }
        }
      }
    }

    // ---- self key of candidate rows: one more online-softmax step, on the tensor cores -----------------------
    // The strip's 16 x 16 block Q K_own^T holds the self logits on its diagonal; the probabilities go back in as a
    // diagonal P block against the strip's own V rows.
    cp_wait<1>();      // the strip's own K/V rows (requested one tile ago) have landed; the next Q may still be in flight
    __syncwarp();
    if (has_cand) {
      float sd[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) { sd[j][0] = sd[j][1] = sd[j][2] = sd[j][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t b0, b1, b2, b3;
        const int kr = (lane & 7) + ((lane >> 4) << 3);
        const int kc = ks * 2 + ((lane >> 3) & 1);
        ldsm_x4(b0, b1, b2, b3, (uint32_t)__cvta_generic_to_shared(wks + swz(kr, kc)));
        mma_bf16_16816(sd[0], qf[ks], b0, b1);
        mma_bf16_16816(sd[1], qf[ks], b2, b3);
      }
      // row g's self key is column g of the first 8-key tile, row g+8's is column g of the second: both sit in the
      // quad's lane t4 == g / 2
      float dsel[2] = {(g & 1) ? sd[0][1] : sd[0][0], (g & 1) ? sd[1][3] : sd[1][2]};
      const int src = (lane & ~3) | (g >> 1);
      const bool mine = (t4 == (g >> 1));
      uint32_t pa[4] = {0u, 0u, 0u, 0u};
      float alpha[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float dot = __shfl_sync(0xffffffffu, dsel[i], src);
        const bool is_cand = segq[i] == -1;
        const float sv_ = is_cand ? (CAP ? scaled_logit(dot, a.sm_scale, a.cap, a.cap_method) : dot * csc) : -INFINITY;
        const float mnew = fmaxf(m[i], sv_);
        const float mns = (mnew == -INFINITY) ? 0.f : mnew;
        alpha[i] = ex2(m[i] - mns);                      // no history yet: 2^-inf = 0; unchanged maximum: 1
        const float p = ex2(sv_ - mns);                  // 0 for rows that are not candidates
        l[i] = l[i] * alpha[i] + p;
        m[i] = mnew;
        const uint32_t pk = (g & 1) ? pack_bf2(0.f, p) : pack_bf2(p, 0.f);   // P rounded to bf16 like every other key
        if (mine) pa[i == 0 ? 0 : 3] = pk;               // A fragment: [g][2t4..], [g+8][2t4..], [g][2t4+8..], [g+8][2t4+8..]
      }
      {
        const float2 a0 = make_float2(alpha[0], alpha[0]), a1 = make_float2(alpha[1], alpha[1]);
#pragma unroll
        for (int j = 0; j < DT; ++j) {
          const float2 x = __fmul2_rn(make_float2(o[j][0], o[j][1]), a0), y = __fmul2_rn(make_float2(o[j][2], o[j][3]), a1);
          o[j][0] = x.x; o[j][1] = x.y; o[j][2] = y.x; o[j][3] = y.y;
        }
      }
#pragma unroll
      for (int jd = 0; jd < DT; jd += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(b0, b1, b2, b3, (uint32_t)__cvta_generic_to_shared(wvs + swz(lane & 15, jd + (lane >> 4))));
        mma_bf16_16816(o[jd], pa, b0, b1);
        mma_bf16_16816(o[jd + 1], pa, b2, b3);
      }
    }
    __syncwarp();
    if (tile + 1 < n_tiles && strip_has_cand(tile + 1)) load_own_kv(tile + 1);
    cp_commit();

    // ---- normalise, stage the strip in its (free) Q buffer, store 16-byte chunks ---------------------------
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float inv = (l[i] == 0.f || segq[i] == 0) ? 0.f : 1.0f / l[i];
      const int lr = g + 8 * i;
#pragma unroll
      for (int j = 0; j < DT; ++j)
        *reinterpret_cast<uint32_t*>(sq + swz(lr, j) + 2 * t4) = pack_bf2(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = lane + 32 * k, r = c >> 3, ch = c & 7;
      const int row = q0 + warp * 16 + r;
      if (row < T)
        *reinterpret_cast<uint4*>(a.out + (trow(row) * a.Hq + h) * DH + ch * 8) =
            *reinterpret_cast<const uint4*>(sq + swz(r, ch));
    }
  }
  cp_wait<0>();
}

template <bool CAP>
phx_status launch_strip(const AttnArgs& a, cudaStream_t stream, std::string& err) {
  static bool attr_set = false;
  if (!attr_set) {
    PHX_CUDA_TRY(cudaFuncSetAttribute(ranker_attention_strip_kernel<CAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, STRIP_SMEM), err);
    attr_set = true;
  }
  dim3 grid(a.Hq, a.B);
  PHX_CUDA_TRY(launch_overlapped(ranker_attention_strip_kernel<CAP>, grid, ATT_THREADS, STRIP_SMEM, stream, a), err);
  return PHX_OK;
}

}  // namespace

phx_status ranker_attention_launch(const AttnArgs& a, cudaStream_t stream, std::string& err) {
  if (a.Hq % a.Hkv != 0) { err = "attention: Hq must be a multiple of Hkv"; return PHX_E_ARG; }
  if (a.B == 0 || a.T == 0) return PHX_OK;
  if (a.B > 65535 || a.Hq > 65535) { err = "attention: batch or head count too large for one launch"; return PHX_E_CAPACITY; }
  {
    const char* force = getenv("PHX_ATTN");
    const bool legacy = force && strcmp(force, "mma") == 0;
    const bool forced_tc = force && (strcmp(force, "tcgen05") == 0 || strcmp(force, "resident") == 0);
    // Histories longer than one key block (128 keys at head dim 64) and head dim 128 go to the streaming tcgen05
    // kernel (measured on B200: 1.5 vs 4.6 ms for the mma.sync kernel at 1024 + 1024 tokens, 16 heads x 128); a
    // history of one key block is the resident-history kernels' case further down.
    const int n_hist = a.hist_len < a.T ? a.hist_len : a.T;
    const bool prefer_tc = forced_tc || a.dh == 128 || n_hist > 128;
    const bool plain = !a.split && a.q_start == 0 && !a.pack.hist_off;   // the tcgen05 kernel's tensor maps assume [B, T] token rows
    if (plain && !legacy && prefer_tc && a.err_flag && ranker_attention_tc_supported(a)) return ranker_attention_tc_launch(a, a.err_flag, stream, err);
  }
  {
    // Head dim 64 with a history of at most 128 keys: the persistent tcgen05 kernel with the history resident and two
    // softmax warpgroups, once there is an item (batch, head) for every SM.  Measured on B200 at the ranking
    // benchmark's shape (B=256, S=128, C=512, 8 heads): 0.140 ms per layer against 0.206 ms for the mma.sync
    // resident-history kernel below (1.2-1.4 against 2.0 ms per step inside the forward), and 0.051 against 0.067 ms at
    // B=64; every byte it touches moves by bulk copies.  PHX_ATTN=strip keeps the mma.sync kernel, PHX_ATTN=pingpong
    // takes this one at any batch size.
    const char* force = getenv("PHX_ATTN");
    const bool forced = force && strcmp(force, "pingpong") == 0;
    const bool fills = !force && (long long)a.B * a.Hq >= 148;
    if ((forced || fills) && a.err_flag && ranker_attention_pingpong_supported(a))
      return ranker_attention_pingpong_launch(a, a.err_flag, stream, err);
  }
  const bool cap = a.cap_method != 0 && a.cap > 0.f;
  {
    // head dim 64 with the whole history in one shared-memory panel: the resident-history kernel
    const char* force = getenv("PHX_ATTN");
    const bool strip_off = force && strcmp(force, "strip") != 0;
    const int n_hist = a.hist_len < a.T ? a.hist_len : a.T;
    // one CTA per (batch, head) walks the request's tiles in sequence: worth it once those CTAs fill the device,
    // while a small batch is better off with one CTA per tile (latency of a single request)
    const bool enough = (long long)a.B * a.Hq >= 148 || (force && strcmp(force, "strip") == 0);
    if (!strip_off && enough && a.dh == 64 && n_hist <= STRIP_HIST) dispatch_note(DK_ATTN_STRIP);
    if (!strip_off && enough && a.dh == 64 && n_hist <= STRIP_HIST) return cap ? launch_strip<true>(a, stream, err) : launch_strip<false>(a, stream, err);
  }
  dispatch_note(DK_ATTN_STREAM);
  switch (a.dh) {
    case 32: return cap ? launch_dh<32, true>(a, stream, err) : launch_dh<32, false>(a, stream, err);
    case 64: return cap ? launch_dh<64, true>(a, stream, err) : launch_dh<64, false>(a, stream, err);
    case 128: return cap ? launch_dh<128, true>(a, stream, err) : launch_dh<128, false>(a, stream, err);
    default: err = "attention: head dim must be 32, 64 or 128"; return PHX_E_ARG;
  }
}

}  // namespace phx
