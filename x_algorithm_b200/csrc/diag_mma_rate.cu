// Diagnostic micro-benchmark of the two resources the GEMM main loop lives on: the tcgen05 pipe and the
// L2 -> shared-memory fill (TMA).  A CTA (or CTA pair) issues the GEMM's MMAs (M=128 per CTA, N=256, K=16, four per
// k-step) over fixed shared-memory tiles; optionally a second warp streams 16 KB TMA tiles into unused parts of the
// stages without synchronising with the MMAs.  Reports the MMA issuer's cycles per k-step, the fill thread's cycles per
// k-step and the kernel time; `python -m x_algorithm_b200.microbench mma` prints them.  No counterpart in the
// reference; it backs the roofline statements about gemm_sm100.cu.  All waits are bounded.
#include <string.h>

#include <string>
#include <vector>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace phx {
namespace {

using namespace sm100;

constexpr int STAGE = 48 * 1024;
constexpr int NST = 4;
constexpr int SMEM = NST * STAGE + 1024 + 512;

template <bool PAIR>
__global__ void __launch_bounds__(128, 1)
rate_kernel(const __grid_constant__ CUtensorMap map, int ksteps, int fill_mode, int depth, int sync_mode, long long fill_rows, int* err,
            unsigned long long* out) {
  extern __shared__ uint8_t raw[];
  const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
  const uint32_t bars = base + NST * STAGE;
  const uint32_t done_bar = bars, fill_bar = bars + 8, slot = bars + 64;
  uint32_t* slot_ptr = reinterpret_cast<uint32_t*>(raw + (slot - smem_u32(raw)));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  volatile int* verr = err;
  // fill smem with a pattern
  for (uint32_t i = threadIdx.x; i < NST * STAGE / 4; i += blockDim.x) {
    uint32_t v = (i * 2654435761u) >> 7;
    v = (v & 0x3fff3fffu) | 0x3c003c00u;  // bf16 values around 1..2 scale, no NaN
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(base + i * 4), "r"(v));
  }
  if (threadIdx.x == 0) {
    mbar_init(done_bar, 1); mbar_init(fill_bar, 1);
    for (int i = 0; i < 16; ++i) mbar_init(bars + 128 + 8 * i, 1);
    for (int i = 0; i < 8; ++i) mbar_init(bars + 256 + 8 * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) { if (PAIR) tmem_alloc_pair(slot, 512); else tmem_alloc(slot, 512); }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  if (warp == 1 && lane == 0 && rank == 0) {
    const uint32_t idesc = make_idesc(PAIR ? 256 : 128, 256);
    const long long t0 = clock64();
    uint32_t ph = 0;
    bool ok = true;
    for (int ks = 0; ks < ksteps && ok; ++ks) {
      const uint32_t a = base + (ks % NST) * STAGE;
      const uint64_t ad = make_smem_desc(a), bd = make_smem_desc(a + 16384);
      const uint32_t d = tmem + ((ks >> 3) & 1) * 256;
      for (int k = 0; k < 4; ++k) {
        if (PAIR) umma_bf16_pair(d, ad + 2 * k, bd + 2 * k, idesc, 1);
        else umma_bf16(d, ad + 2 * k, bd + 2 * k, idesc, 1);
      }
      if (sync_mode == 0) {
        if ((ks & 7) == 7) {
          if (PAIR) umma_commit_pair(done_bar, 1); else umma_commit(done_bar);
          if (ks >= 15) { ok = mbar_wait(done_bar, ph, verr); ph ^= 1; }
        }
      } else {
        // one commit per k-step on a ring of 8 barriers; mode 2 also waits for the commit of 4 k-steps ago
        const uint32_t rb = bars + 256 + 8 * (ks & 7);
        if (PAIR) umma_commit_pair(rb, 1); else umma_commit(rb);
        if (sync_mode == 2 && ks >= 4) ok = mbar_wait(bars + 256 + 8 * ((ks - 4) & 7), ((ks - 4) >> 3) & 1, verr);
      }
    }
    // drain
    if (ok) {
      if (sync_mode == 0) { if (ksteps >= 16) { ok = mbar_wait(done_bar, ph, verr); ph ^= 1; } }
      else ok = mbar_wait(bars + 256 + 8 * ((ksteps - 1) & 7), ((ksteps - 1) >> 3) & 1, verr);
    }
    const long long t1 = clock64();
    out[blockIdx.x] = (unsigned long long)(t1 - t0);
  }
  if (warp == 0 && lane == 0 && fill_mode != 0) {
    // unsynchronised fill traffic: 16 KB TMA tiles (128 rows x 64 cols) into bytes 32768.. of the stages; `depth` k-steps in flight
    const int tiles_per_k = fill_mode;
    int r = (int)((blockIdx.x * 4096ll) % fill_rows);
    bool ok = true;
    int slot_i = 0, slot_w = 0; uint32_t ph_w = 0;
    const long long f0 = clock64();
    for (int ks = 0; ks < ksteps + depth && ok; ++ks) {
      if (ks >= depth) { ok = mbar_wait(bars + 128 + 8 * slot_w, ph_w, verr); if (++slot_w == depth) { slot_w = 0; ph_w ^= 1; } }
      if (ks < ksteps && ok) {
        const uint32_t fb = bars + 128 + 8 * slot_i;
        if (++slot_i == depth) slot_i = 0;
        mbar_expect_tx(fb, tiles_per_k * 16384);
        for (int t = 0; t < tiles_per_k; ++t) {
          tma_load_2d(base + ((ks + 2) & 3) * STAGE + 32768, &map, fb, ((ks * 3 + t) & 7) * 64, r);
          r += 128; if (r >= fill_rows) r -= (int)fill_rows;
        }
      }
    }
    out[148 + blockIdx.x] = (unsigned long long)(clock64() - f0);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  if (warp == 1) { tc_fence_after(); if (PAIR) tmem_dealloc_pair(tmem, 512); else tmem_dealloc(tmem, 512); }
}


template <bool PAIR>
phx_status diag_run(const CUtensorMap& map, int ksteps, int fill_tiles, int depth, int sync_mode, long long fill_rows, float* ms_out,
                    double* mma_cyc, double* fill_cyc, std::string& err) {
  int* errf = nullptr; unsigned long long* out = nullptr;
  PHX_CUDA_TRY(cudaMalloc(&errf, 4), err);
  PHX_CUDA_TRY(cudaMalloc(&out, 296 * 8), err);
  cudaMemset(errf, 0, 4); cudaMemset(out, 0, 296 * 8);
  auto kern = rate_kernel<PAIR>;
  PHX_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM), err);
  cudaLaunchConfig_t lc; memset(&lc, 0, sizeof(lc));
  cudaLaunchAttribute at[1];
  lc.blockDim = dim3(128); lc.gridDim = dim3(148); lc.dynamicSmemBytes = SMEM;
  if (PAIR) { at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1; lc.attrs = at; lc.numAttrs = 1; }
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  float best = 1e30f;
  phx_status st = PHX_OK;
  for (int rep = 0; rep < 2 && st == PHX_OK; ++rep) {
    cudaEventRecord(e0);
    cudaError_t le = cudaLaunchKernelEx(&lc, kern, map, ksteps, fill_tiles, depth, sync_mode, fill_rows, errf, out);
    cudaEventRecord(e1);
    cudaError_t ce = cudaEventSynchronize(e1);
    if (le != cudaSuccess || ce != cudaSuccess) { err = std::string("diag kernel: ") + cudaGetErrorString(le != cudaSuccess ? le : ce); st = PHX_E_CUDA; break; }
    float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < best) best = ms;
  }
  if (st == PHX_OK) {
    int herr = 0; cudaMemcpy(&herr, errf, 4, cudaMemcpyDeviceToHost);
    if (herr) { err = "a bounded device-side wait ran out (diagnostic kernel)"; st = PHX_E_TIMEOUT; }
    std::vector<unsigned long long> h(296);
    cudaMemcpy(h.data(), out, 296 * 8, cudaMemcpyDeviceToHost);
    double sum = 0, fsum = 0; int n = 0;
    for (int i = 0; i < 148; ++i) if (h[i]) { sum += (double)h[i]; ++n; }
    for (int i = 148; i < 296; ++i) fsum += (double)h[i];
    *mma_cyc = n ? sum / n / ksteps : 0.0;
    *fill_cyc = fill_tiles ? fsum / 148 / ksteps : 0.0;
    *ms_out = best;
  }
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  cudaFree(errf); cudaFree(out);
  return st;
}

}  // namespace
}  // namespace phx

using namespace phx;

extern "C" phx_status phx_diag_mma_rate(int32_t device, int32_t pair, int32_t ksteps, int32_t fill_tiles_per_kstep, int32_t sync_mode,
                                        float* ms_out, double* mma_cycles_per_kstep, double* fill_cycles_per_kstep) {
  std::string err;
  if (!ms_out || !mma_cycles_per_kstep || !fill_cycles_per_kstep || ksteps < 16 || ksteps % 8 != 0 || fill_tiles_per_kstep < 0 ||
      fill_tiles_per_kstep > 3 || sync_mode < 0 || sync_mode > 2) {
    set_global_error("phx_diag_mma_rate: bad argument (ksteps a multiple of 8, >= 16; 0..3 fill tiles; sync mode 0..2)");
    return PHX_E_ARG;
  }
  if (cudaSetDevice(device) != cudaSuccess) { set_global_error("cudaSetDevice failed"); return PHX_E_CUDA; }
  const long long rows = 1 << 18;   // 256 K rows x 512 cols bf16 = 256 MB: larger than L2
  bf16* buf = nullptr;
  if (cudaMalloc(&buf, (size_t)rows * 512 * 2) != cudaSuccess) { set_global_error("phx_diag_mma_rate: cudaMalloc failed"); return PHX_E_CUDA; }
  cudaMemset(buf, 0x3c, (size_t)rows * 512 * 2);
  CUtensorMap map;
  phx_status st = sm100::make_map(&map, buf, rows, 512, 128, err);
  if (st == PHX_OK)
    st = pair ? diag_run<true>(map, ksteps, fill_tiles_per_kstep, 8, sync_mode, rows, ms_out, mma_cycles_per_kstep, fill_cycles_per_kstep, err)
              : diag_run<false>(map, ksteps, fill_tiles_per_kstep, 8, sync_mode, rows, ms_out, mma_cycles_per_kstep, fill_cycles_per_kstep, err);
  cudaFree(buf);
  if (st) set_global_error(err);
  return st;
}
