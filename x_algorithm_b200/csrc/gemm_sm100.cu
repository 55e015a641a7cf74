// bf16 GEMM for the Linear layers of the Phoenix trunk (phoenix/xrex/models/linear_layer.py:52-91)
// on Blackwell tensor cores: C[M,N] = epilogue(A[M,K] @ Wt[N,K]^T), fp32 accumulation in TMEM.
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer: A tile 128x64 and W tile BNx64 (bf16, 128-byte swizzle) per k-step
//               into a ring of shared-memory stages (cp.async.bulk.tensor + mbarrier tx count)
//   warp 1      MMA issuer: one lane issues tcgen05.mma (M=128, N=BN, K=16) x4 per stage into one
//               of two TMEM accumulators, tcgen05.commit releases the stage / publishes the tile
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (each warp its 32-lane quadrant),
//               fused epilogue (store | +residual | GELU-tanh), bf16 stores; overlaps the next
//               tile's main loop through the second accumulator
// Every mbarrier wait is bounded by wall time; on expiry the kernel raises *err_flag and unwinds.
#include "common.cuh"

namespace phx {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s

template <int BN>
struct Cfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // +1024 alignment slack
  static constexpr int TMEM_COLS = 2 * BN;                                    // two accumulators
};

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when the limit ran out or another role already raised the flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* err_flag) {
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((it & 0x3FF) == 0x3FF) {
      if (*err_flag != 0) return false;
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) { *err_flag = 1; __threadfence(); return false; }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread = lane = row)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row
// groups 1024 bytes apart (stride byte offset), descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);          // start address, bits [0,14)
  d |= (uint64_t)(0) << 16;                             // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                               // descriptor version
  d |= (uint64_t)2 << 61;                               // layout: SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16: D fp32, A/B bf16, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) {
  return (1u << 4)                       // D format: f32
         | (1u << 7)                     // A format: bf16
         | (1u << 10)                    // B format: bf16
         | ((uint32_t)(N >> 3) << 17)    // N / 8
         | ((uint32_t)(M >> 4) << 24);   // M / 16
}

template <int EPI>
__device__ __forceinline__ void epilogue_chunk(const uint32_t* acc, bf16* c_row, const bf16* r_row, int col0, int N) {
  // 32 fp32 accumulators -> 32 bf16, 16-byte stores; N % 8 == 0 is guaranteed by the host
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    int col = col0 + g * 8;
    if (col >= N) break;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = round_bf(__uint_as_float(acc[g * 8 + i]));  // Linear output is bf16
    if (EPI == EPI_RESIDUAL) {
      uint4 rr = *reinterpret_cast<const uint4*>(r_row + col);
      float2 a = unpack_bf2(rr.x), b = unpack_bf2(rr.y), c = unpack_bf2(rr.z), d = unpack_bf2(rr.w);
      v[0] += a.x; v[1] += a.y; v[2] += b.x; v[3] += b.y; v[4] += c.x; v[5] += c.y; v[6] += d.x; v[7] += d.y;
    } else if (EPI == EPI_GELU) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = gelu_tanh_f(v[i]);
    }
    uint4 o;
    o.x = pack_bf2(v[0], v[1]); o.y = pack_bf2(v[2], v[3]); o.z = pack_bf2(v[4], v[5]); o.w = pack_bf2(v[6], v[7]);
    *reinterpret_cast<uint4*>(c_row + col) = o;
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    bf16* C, const bf16* R, long long M, int N, int K, int* err_flag) {
  // C and R may alias (in-place residual update): each thread reads its R chunk before writing the same C chunk
  using cfg = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  const uint32_t bars = smem_base + cfg::STAGES * cfg::STAGE_BYTES;
  // barrier slots (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then the TMEM slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (cfg::STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * cfg::STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * cfg::STAGES + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * cfg::STAGES + 4);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (N + BN - 1) / BN;
  const long long m_tiles = (M + BM - 1) / BM;
  const long long total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + BK - 1) / BK;
  volatile int* verr = err_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < cfg::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 128); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int n_blk = (int)(tile % n_tiles);
        const long long m_blk = tile / n_tiles;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, verr)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * cfg::STAGE_BYTES;
          const uint32_t b_dst = a_dst + cfg::A_BYTES;
          mbar_expect_tx(full_bar(stage), cfg::STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, full_bar(stage), kb * BK, (int)(m_blk * BM));
          tma_load_2d(b_dst, &map_b, full_bar(stage), kb * BK, n_blk * BN);
          if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      int stage = 0; uint32_t phase = 0;
      uint32_t it = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, verr)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, verr)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * cfg::STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(a_src);
          const uint64_t bdesc = make_smem_desc(a_src + cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing 16 elements along K inside the 128-byte swizzle row = +32 bytes = +2 in the address field
            umma_bf16(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb | k) != 0);
          }
          umma_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
          if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(tfull_bar(acc));  // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    uint32_t it = 0;
    bool ok = true;
    for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      const int n_blk = (int)(tile % n_tiles);
      const long long m_blk = tile / n_tiles;
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), acc_phase, verr)) { ok = false; break; }
      tc_fence_after();
      const long long row = m_blk * BM + quad * 32 + lane;
      const bool row_ok = row < M;
      bf16* c_row = C + row * (long long)N;
      const bf16* r_row = (EPI == EPI_RESIDUAL) ? (R + row * (long long)N) : nullptr;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        const int col0 = n_blk * BN + c * 32;
        if (row_ok && col0 < N) epilogue_chunk<EPI>(r, c_row, r_row, col0, N);
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));
    }
  }

  // ---------------- teardown ----------------
  if (*verr != 0) __nanosleep(1000000);  // error path: let in-flight bulk copies land before the CTA retires
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, cfg::TMEM_COLS);
  }
}

// ---- tensor map creation through the runtime's driver entry point (no libcuda link needed) ---------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn(std::string& err) {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || p == nullptr) {
    err = std::string("cudaGetDriverEntryPoint(cuTensorMapEncodeTiled) failed: ") + cudaGetErrorString(e);
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// 2-D bf16 tensor [rows, cols] row-major; box = [box_rows, 64 cols], 128-byte swizzle, zero OOB fill
phx_status make_map(CUtensorMap* map, const bf16* ptr, int64_t rows, int64_t cols, int box_rows, std::string& err) {
  EncodeTiledFn fn = get_encode_fn(err);
  if (!fn) return PHX_E_CUDA;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (cols % 8) != 0) {
    err = "gemm: operand pointer must be 16-byte aligned and K a multiple of 8";
    return PHX_E_ARG;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<bf16*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    err = "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r);
    return PHX_E_CUDA;
  }
  return PHX_OK;
}

template <int BN, int EPI>
phx_status launch_t(const GemmPlan& p, bf16* C, const bf16* R, int64_t M, int* err_flag, int num_sms,
                    cudaStream_t stream, std::string& err) {
  using cfg = Cfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    PHX_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      cfg::SMEM_BYTES), err);
    attr_set = true;
  }
  const long long tiles = ((M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int grid = (int)(tiles < num_sms ? tiles : num_sms);
  if (grid <= 0) return PHX_OK;
  gemm_tcgen05_kernel<BN, EPI><<<grid, GEMM_THREADS, cfg::SMEM_BYTES, stream>>>(p.map_a, p.map_b, C, R, M, p.N, p.K,
                                                                               err_flag);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

// ---- SIMT cross-check GEMM --------------------------------------------------------------------------
template <int EPI>
__global__ void gemm_simt_kernel(const bf16* __restrict__ A, const bf16* __restrict__ Wt, bf16* C,
                                 const bf16* R, long long M, int N, int K) {
  __shared__ float sa[32][33];
  __shared__ float sb[32][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const long long row = (long long)blockIdx.y * 32 + ty;
  const int col = blockIdx.x * 32 + tx;
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += 32) {
    sa[ty][tx] = (row < M && k0 + tx < K) ? bf2f(A[row * K + k0 + tx]) : 0.f;
    const int wr = blockIdx.x * 32 + ty;
    sb[ty][tx] = (wr < N && k0 + tx < K) ? bf2f(Wt[(long long)wr * K + k0 + tx]) : 0.f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 32; ++k) acc += sa[ty][k] * sb[tx][k];
    __syncthreads();
  }
  if (row < M && col < N) {
    float v = round_bf(acc);
    if (EPI == EPI_RESIDUAL) v += bf2f(R[row * N + col]);
    else if (EPI == EPI_GELU) v = gelu_tanh_f(v);
    C[row * N + col] = f2bf(v);
  }
}

}  // namespace

phx_status gemm_plan_create(GemmPlan* plan, const bf16* A, const bf16* Wt, int64_t rows_max, int N, int K,
                            std::string& err) {
  if (N % 8 != 0 || K % 8 != 0 || N <= 0 || K <= 0 || rows_max <= 0) {
    err = "gemm: N and K must be positive multiples of 8";
    return PHX_E_ARG;
  }
  plan->A = A; plan->Wt = Wt; plan->rows_max = rows_max; plan->N = N; plan->K = K;
  plan->BN = (N % 256 == 0) ? 256 : 128;
  phx_status s = make_map(&plan->map_a, A, rows_max, K, BM, err);
  if (s != PHX_OK) return s;
  s = make_map(&plan->map_b, Wt, N, K, plan->BN, err);
  if (s != PHX_OK) return s;
  plan->ready = true;
  return PHX_OK;
}

phx_status gemm_launch(const GemmPlan& p, bf16* C, const bf16* R, int64_t M, int epilogue, int* err_flag,
                       int num_sms, cudaStream_t stream, std::string& err) {
  if (!p.ready || M > p.rows_max) { err = "gemm: plan not ready or M exceeds plan rows"; return PHX_E_ARG; }
  if (epilogue == EPI_RESIDUAL && R == nullptr) { err = "gemm: residual epilogue needs R"; return PHX_E_ARG; }
  if (p.BN == 256) {
    switch (epilogue) {
      case EPI_STORE: return launch_t<256, EPI_STORE>(p, C, R, M, err_flag, num_sms, stream, err);
      case EPI_RESIDUAL: return launch_t<256, EPI_RESIDUAL>(p, C, R, M, err_flag, num_sms, stream, err);
      case EPI_GELU: return launch_t<256, EPI_GELU>(p, C, R, M, err_flag, num_sms, stream, err);
    }
  } else {
    switch (epilogue) {
      case EPI_STORE: return launch_t<128, EPI_STORE>(p, C, R, M, err_flag, num_sms, stream, err);
      case EPI_RESIDUAL: return launch_t<128, EPI_RESIDUAL>(p, C, R, M, err_flag, num_sms, stream, err);
      case EPI_GELU: return launch_t<128, EPI_GELU>(p, C, R, M, err_flag, num_sms, stream, err);
    }
  }
  err = "gemm: unknown epilogue";
  return PHX_E_ARG;
}

phx_status gemm_simt_launch(const bf16* A, const bf16* Wt, bf16* C, const bf16* R, int64_t M, int N, int K,
                            int epilogue, cudaStream_t stream, std::string& err) {
  dim3 block(32, 32);
  dim3 grid((N + 31) / 32, (unsigned)((M + 31) / 32));
  if (grid.y > 65535) {
    // split rows so gridDim.y stays legal
    const int64_t chunk = 65535LL * 32;
    for (int64_t m0 = 0; m0 < M; m0 += chunk) {
      int64_t mm = (M - m0 < chunk) ? (M - m0) : chunk;
      phx_status s = gemm_simt_launch(A + m0 * K, Wt, C + m0 * N, R ? R + m0 * N : nullptr, mm, N, K, epilogue,
                                      stream, err);
      if (s != PHX_OK) return s;
    }
    return PHX_OK;
  }
  switch (epilogue) {
    case EPI_STORE: gemm_simt_kernel<EPI_STORE><<<grid, block, 0, stream>>>(A, Wt, C, R, M, N, K); break;
    case EPI_RESIDUAL: gemm_simt_kernel<EPI_RESIDUAL><<<grid, block, 0, stream>>>(A, Wt, C, R, M, N, K); break;
    case EPI_GELU: gemm_simt_kernel<EPI_GELU><<<grid, block, 0, stream>>>(A, Wt, C, R, M, N, K); break;
    default: err = "gemm: unknown epilogue"; return PHX_E_ARG;
  }
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

}  // namespace phx
