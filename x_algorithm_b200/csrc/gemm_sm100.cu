// bf16 GEMM for the Linear layers of the Phoenix trunk (phoenix/xrex/models/linear_layer.py:52-91)
// on Blackwell tensor cores: C[M,N] = epilogue(A[M,K] @ Wt[N,K]^T), fp32 accumulation in TMEM.
//
// Persistent kernel, one CTA per SM, 64 + 128 x NG threads (NG = epilogue groups: 2 or 4):
//   warp 0      TMA producer: A tile 128x64 and W tile per k-step (bf16, 128-byte swizzle) into a ring of
//               shared-memory stages (cp.async.bulk.tensor + mbarrier tx count)
//   warp 1      MMA issuer: one lane issues tcgen05.mma (N=BN, K=16) x4 per stage into one of two TMEM
//               accumulators, tcgen05.commit releases the stage / publishes the tile
//   warps 2..   epilogue, NG groups of four warps: tcgen05.ld the finished accumulator (each warp its
//               32-lane quadrant) in 64-column slabs, fused op (store | +residual | GELU-tanh | RoPE | RMSNorm
//               scale), bf16 slab staged in swizzled shared memory and written by one TMA bulk store; the
//               residual slab is fetched by TMA ahead of its use; overlaps the next tile's main loop through
//               the second accumulator
// PAIR variant (cta_group::2): the two CTAs of a cluster work on one 256 x BN tile.  Each loads its own 128 rows of
// A and its own half of the W tile, the even CTA issues one MMA (M=256) that reads both shared memories and
// writes each CTA's 128 rows into that CTA's TMEM, and each CTA runs the epilogue on its own rows.  Operand bytes
// per CTA per k-step fall from 128+BN to 128+BN/2 rows: the GEMM is bound by that shared-memory fill.
// Every mbarrier wait is bounded by wall time; on expiry the kernel raises *err_flag and unwinds.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace phx {

namespace {

using namespace sm100;
constexpr int BM = 128;
// threads: TMA warp, MMA warp, NG epilogue groups of four warps
constexpr int gemm_threads(int ng) { return 64 + ng * 128; }

template <int BN, bool PAIR, int NG>
struct Cfg {
  static_assert(NG == 2 || (NG == 4 && PAIR), "four epilogue groups need the smaller stages of a CTA pair");
  static constexpr int STAGES = PAIR ? 5 : 4;
  // output slab buffers, NSLAB / NG per epilogue group
  static constexpr int NSLAB = NG == 4 ? 4 : (PAIR ? ((BN == 256) ? 4 : 6) : ((BN == 256) ? 2 : 6));
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;   // rows of the W tile this CTA loads
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + NSLAB * (128 * 64 * 2) + BAR_BYTES + 1024;  // + slabs, +1024 alignment slack
  static constexpr int TMEM_COLS = 2 * BN;                                    // two accumulators
};

// ---- epilogue helpers -----------------------------------------------------------------------------
constexpr int SLAB_COLS = 64;                 // one output slab = 128 rows x 64 bf16 columns = 128-byte rows
constexpr int SLAB_BYTES = BM * SLAB_COLS * 2;

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// named barrier `id` over the 128 threads of one epilogue group, AND-reducing a per-thread flag: every thread
// always arrives, so a thread that gave up on a bounded wait can never leave the others parked here
__device__ __forceinline__ bool epi_barrier_and(bool ok, int id) {
  uint32_t out;
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.and.pred p, %2, 128, q;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(out) : "r"((uint32_t)ok), "r"(id) : "memory");
  return out != 0;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int BN, int EPI, bool PAIR, int NG>
__global__ void __launch_bounds__(gemm_threads(NG), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_r,
                    GemmRope rope, GemmNorm norm, long long M, int N, int K, int* err_flag,
                    unsigned long long* counters) {
  // C and R may be the same buffer (in-place residual update): a slab is fetched before it is written back,
  // and no other CTA touches the tile.
  using cfg = Cfg<BN, PAIR, NG>;
  constexpr int SLABS = BN / SLAB_COLS;
  // epilogue threads that drain one accumulator (a tile with fewer slabs than groups is shared by SLABS groups)
  constexpr int DRAIN_THREADS = (SLABS < NG ? SLABS : NG) * 128 * (PAIR ? 2 : 1);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  const uint32_t slab_base = smem_base + cfg::STAGES * cfg::STAGE_BYTES;   // output slab buffers
  const uint32_t bars = slab_base + cfg::NSLAB * SLAB_BYTES;
  // barrier slots (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], res[NSLAB]; then the TMEM slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (cfg::STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * cfg::STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * cfg::STAGES + 2 + a); };
  auto res_bar = [&](int b) { return bars + 8u * (2 * cfg::STAGES + 4 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * cfg::STAGES + 4 + cfg::NSLAB);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (counters && blockIdx.x == 0 && threadIdx.x == 0) counters[3] = globaltimer_ns();   // diagnostics: kernel entry
  constexpr int TILE_M = PAIR ? 2 * BM : BM;          // rows of one work tile (of the CTA pair)
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u; // 0 = the CTA that issues the pair's MMAs
  const long long first_tile = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const long long tile_step = PAIR ? (gridDim.x >> 1) : gridDim.x;
  const int n_tiles = (N + BN - 1) / BN;
  const long long m_tiles = (M + TILE_M - 1) / TILE_M;
  const long long total_tiles = m_tiles * n_tiles;
  const int k_blocks = (K + BK - 1) / BK;
  volatile int* verr = err_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < cfg::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    // a pair's accumulators are drained by the epilogue threads of both CTAs, counted on the issuing CTA
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), DRAIN_THREADS); }
    for (int a = 0; a < cfg::NSLAB; ++a) mbar_init(res_bar(a), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) tmem_alloc_pair(tmem_slot, cfg::TMEM_COLS);
    else tmem_alloc(tmem_slot, cfg::TMEM_COLS);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Programmatic dependent launch: everything above (barriers, tensor memory, cluster hand-shake) touched no global
  // data, so it may run while the kernel in front of this one on the stream is still finishing.  From here on the
  // kernel reads what its predecessor wrote: wait for it (a no-op for a launch without the attribute), and let the
  // kernel behind start its own set-up.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (long long tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
        const int n_blk = (int)(tile % n_tiles);
        const long long m_blk = tile / n_tiles;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, verr)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * cfg::STAGE_BYTES;
          const uint32_t b_dst = a_dst + cfg::A_BYTES;
          if (PAIR) {
            // both CTAs' bytes are counted on the issuing CTA's barrier
            const uint32_t bar0 = mapa_shared(full_bar(stage), 0);
            if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * cfg::STAGE_BYTES);
            tma_load_2d_pair(a_dst, &map_a, bar0, kb * BK, (int)(m_blk * TILE_M + rank * BM));
            tma_load_2d_pair(b_dst, &map_b, bar0, kb * BK, n_blk * BN + (int)rank * cfg::B_ROWS);
          } else {
            mbar_expect_tx(full_bar(stage), cfg::STAGE_BYTES);
            tma_load_2d(a_dst, &map_a, full_bar(stage), kb * BK, (int)(m_blk * BM));
            tma_load_2d(b_dst, &map_b, full_bar(stage), kb * BK, n_blk * BN);
          }
          if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (PAIR && ok) {
        // the issuing CTA releases stages in this CTA by remote arrivals: all of them must have landed before
        // this CTA may retire
        for (int s = 0; s < cfg::STAGES; ++s) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, verr)) break;
          if (++stage == cfg::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // One thread, and the pipe only stays fed if this loop is short: the thread shares its scheduler with four
    // epilogue warps, so every instruction here costs several cycles of wall time.  Stage addresses and descriptors
    // are carried as running values (no per-step address arithmetic), the wait counters exist only when asked for.
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc(TILE_M, BN);
      constexpr uint64_t DESC_STEP = (uint64_t)(cfg::STAGE_BYTES >> 4);    // descriptor address field: bytes / 16
      const uint64_t adesc0 = make_smem_desc(smem_base);
      const uint64_t bdesc0 = make_smem_desc(smem_base + cfg::A_BYTES);
      uint64_t adesc = adesc0, bdesc = bdesc0;
      uint32_t full_addr = full_bar(0), empty_addr = empty_bar(0);
      int stage = 0; uint32_t phase = 0;
      uint32_t it = 0;
      bool ok = true;
      long long cnt_tempty = 0, cnt_full = 0;
      const bool timed = counters != nullptr;
      const long long t_start = timed ? clock64() : 0;
      if (timed && blockIdx.x == 0) counters[4] = globaltimer_ns();   // first MMA wait
      for (long long tile = first_tile; tile < total_tiles && ok; tile += tile_step, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        long long c0 = timed ? clock64() : 0;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, verr)) { ok = false; break; }
        if (timed) cnt_tempty += clock64() - c0;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (timed) c0 = clock64();
          if (!mbar_wait(full_addr, phase, verr)) { ok = false; break; }
          if (timed) cnt_full += clock64() - c0;
          tc_fence_after();
          // advancing 16 elements along K inside the 128-byte swizzle row = +32 bytes = +2 in the address field
          if (PAIR) {
            umma_bf16_pair(tmem_d, adesc, bdesc, idesc, kb != 0);
            umma_bf16_pair(tmem_d, adesc + 2, bdesc + 2, idesc, 1);
            umma_bf16_pair(tmem_d, adesc + 4, bdesc + 4, idesc, 1);
            umma_bf16_pair(tmem_d, adesc + 6, bdesc + 6, idesc, 1);
            umma_commit_pair(empty_addr, 3);   // stage reusable (in both CTAs) once these MMAs have read it
          } else {
            umma_bf16(tmem_d, adesc, bdesc, idesc, kb != 0);
            umma_bf16(tmem_d, adesc + 2, bdesc + 2, idesc, 1);
            umma_bf16(tmem_d, adesc + 4, bdesc + 4, idesc, 1);
            umma_bf16(tmem_d, adesc + 6, bdesc + 6, idesc, 1);
            umma_commit(empty_addr);
          }
          adesc += DESC_STEP; bdesc += DESC_STEP; full_addr += 8; empty_addr += 8;
          if (++stage == cfg::STAGES) {
            stage = 0; phase ^= 1;
            adesc = adesc0; bdesc = bdesc0; full_addr = full_bar(0); empty_addr = empty_bar(0);
          }
        }
        if (ok) {  // accumulator complete
          if (PAIR) umma_commit_pair(tfull_bar(acc), 3); else umma_commit(tfull_bar(acc));
        }
      }
      if (timed) {   // diagnostic: where the MMA issuer spent its time (cycles summed over CTAs)
        atomicAdd(&counters[0], (unsigned long long)(clock64() - t_start));
        atomicAdd(&counters[1], (unsigned long long)cnt_full);
        atomicAdd(&counters[2], (unsigned long long)cnt_tempty);
        if (blockIdx.x == 0) counters[5] = globaltimer_ns();   // last MMA issued
      }
    }
  } else {
    // ---------------- epilogue (warps 2..: NG groups of four warps) ----------------
    // Work item = one 64-column slab of a tile; group gidx takes the items with q % NG == gidx and owns NB
    // slab buffers, an issuing thread and named barrier 1 + gidx.  Per item: TMEM -> registers -> fused op
    // -> swizzled shared-memory slab -> one TMA bulk store.  The residual slab arrives by TMA into the same
    // buffer (up to NB - 1 items ahead, at least one) and is updated in place.
    constexpr int NB = cfg::NSLAB / NG;
    constexpr bool RES = (EPI == EPI_RESIDUAL);
    constexpr int DIST = NB - 1;                        // residual prefetch distance (items of this group)
    const int ew = warp - 2;
    const int gidx = ew >> 2;
    const int quad = warp & 3;                          // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    const bool issuer = ((ew & 3) == 0 && lane == 0);
    const long long my_tiles = (total_tiles > first_tile) ? (total_tiles - first_tile + tile_step - 1) / tile_step : 0;
    // the accumulator-drained signal goes to the CTA that issues the MMAs
    const uint32_t tempty0 = PAIR ? mapa_shared(tempty_bar(0), 0) : tempty_bar(0);
    const uint32_t tempty1 = PAIR ? mapa_shared(tempty_bar(1), 0) : tempty_bar(1);
    auto release_acc = [&](uint32_t a) {
      tc_fence_before();
      if (PAIR) mbar_arrive_cluster(a ? tempty1 : tempty0);
      else mbar_arrive(a ? tempty1 : tempty0);
    };
    const long long total_items = my_tiles * SLABS;
    const long long my_items = (total_items > gidx) ? (total_items - gidx + NG - 1) / NG : 0;
    const uint32_t gslab = slab_base + gidx * NB * SLAB_BYTES;
    auto coords = [&](long long i, long long& m0, int& c0) {   // i = item index inside this group
      const long long q = (long long)NG * i + gidx;
      const long long tile = first_tile + (q / SLABS) * tile_step;
      m0 = (tile / n_tiles) * TILE_M + rank * BM;
      c0 = (int)(tile % n_tiles) * BN + (int)(q % SLABS) * SLAB_COLS;
    };
    auto issue_res = [&](long long i) {
      long long m1; int c1; coords(i, m1, c1);
      const int bi = (int)(i % NB);
      mbar_expect_tx(res_bar(gidx * NB + bi), SLAB_BYTES);
      tma_load_2d(gslab + bi * SLAB_BYTES, &map_r, res_bar(gidx * NB + bi), c1, (int)m1);
    };
    if (RES && issuer) {
      for (int i = 0; i < DIST && i < my_items; ++i) issue_res(i);
    }
    float rstd = 1.0f;   // 1/rms of this thread's row, refreshed at each tile
    for (long long i = 0; i < my_items; ++i) {
      const long long q = (long long)NG * i + gidx;
      const int s = (int)(q % SLABS);
      const uint32_t it = (uint32_t)(q / SLABS), acc = it & 1, acc_phase = (it >> 1) & 1;
      const int bi = (int)(i % NB);
      const uint32_t slab = gslab + bi * SLAB_BYTES;
      long long m0; int c0; coords(i, m0, c0);
      const bool first_of_tile = (s < NG);              // this group's first slab of the tile
      // RMSNorm folded into this GEMM: the row's 1/rms comes from the sum of squares its producer left behind
      // (partials in fixed slots, summed in slot order: deterministic), the gain is folded into the weights.
      // Read once per tile, before the wait on the accumulator, so the loads hide behind it.
      float4 ssa = make_float4(0.f, 0.f, 0.f, 0.f), ssb = ssa;   // up to 8 partials, summed after the wait below
      float ss_rest = 0.f;
      const bool need_rstd = !RES && norm.ss_in != nullptr && first_of_tile;
      if (need_rstd) {
        const long long row = m0 + row_in_tile;
        if (row < M) {
          const float* sp = norm.ss_in + row * norm.slots_in;
          if (norm.slots_in == 8) {
            ssa = __ldg(reinterpret_cast<const float4*>(sp));
            ssb = __ldg(reinterpret_cast<const float4*>(sp + 4));
          } else if (norm.slots_in == 4) {
            ssa = __ldg(reinterpret_cast<const float4*>(sp));
          } else {
            for (int t = 0; t < norm.slots_in; ++t) ss_rest += __ldg(sp + t);
          }
        }
      }
      const bool last_of_tile = (s + NG >= SLABS);      // ... and its last
      if (RES && issuer && i + DIST < my_items) {
        // the buffer of item i + DIST was last used by item i - 1: its store must have drained
        bulk_wait_read<0>();
        issue_res(i + DIST);
      }
      bool ok = true;
      if (first_of_tile) ok = mbar_wait(tfull_bar(acc), acc_phase, verr);
      if (RES && ok) ok = mbar_wait(res_bar(gidx * NB + bi), (uint32_t)((i / NB) & 1), verr);
      ok = __all_sync(0xffffffffu, ok);
      if (need_rstd) {   // slot order: deterministic
        float ss = ss_rest;
        ss += ssa.x; ss += ssa.y; ss += ssa.z; ss += ssa.w; ss += ssb.x; ss += ssb.y; ss += ssb.z; ss += ssb.w;
        rstd = rsqrtf(ss * norm.inv_d + norm.eps);
      }
      const uint32_t row_addr = slab + row_in_tile * 128;
      const int sw = row_in_tile & 7;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16) + s * SLAB_COLS;
      if (!RES) {
        // the store that last read this buffer (item i - NB of this group) must have drained before it is rewritten
        if (issuer) bulk_wait_read<NB - 1>();
        ok = epi_barrier_and(ok, 1 + gidx);
      }
      if (ok) {
        tc_fence_after();
        if (EPI == EPI_ROPE) {
          // RoPE on the q / k head parts of this slab (layers.py:52-67, 784-788), pairs (j, j + dh/2), in two
          // passes of 16 pairs so that only 32 values are live: head dim 64 = one part per slab, pass p rotates
          // columns [16p, 16p+16) against [32+16p, 48+16p); head dim 32 = pass p is the slab's p-th part.
          const long long row = m0 + row_in_tile + rope.row_offset;
          int pos = rope.pos_cap;                       // split layout: the candidate block sits at the cap
          if (rope.pos_rows) {                          // packed rows: the position comes with the row
            pos = row < M + rope.row_offset ? rope.pos_rows[row] : 0;
          } else if (rope.split_rows == 0 || row < rope.split_rows) {
            const int t = (int)(row % rope.T);
            pos = t < rope.pos_cap ? t : rope.pos_cap;
          }
          const bool d64 = (rope.dh == 64);
          const int half = rope.dh >> 1;
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int lo_col = d64 ? 16 * p : 32 * p;
            const int hi_col = d64 ? 32 + 16 * p : 32 * p + 16;
            uint32_t rl[16], rh[16];
            tmem_ld16_nowait(taddr + lo_col, rl);
            tmem_ld16_nowait(taddr + hi_col, rh);
            tmem_ld_wait();
            if (p == 1 && last_of_tile) release_acc(acc);
            const int kind = d64 ? (c0 >> 6) % rope.group : ((c0 >> 5) + p) % rope.group;
            float lo[16], hi[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) {   // Linear output is bf16
              lo[k] = round_bf(__uint_as_float(rl[k]) * rstd);
              hi[k] = round_bf(__uint_as_float(rh[k]) * rstd);
            }
            if (kind <= rope.g) {   // q or k part (v parts pass through)
              const float4* c4 = reinterpret_cast<const float4*>(rope.cos_tab + (long long)pos * half + (d64 ? 16 * p : 0));
              const float4* s4 = reinterpret_cast<const float4*>(rope.sin_tab + (long long)pos * half + (d64 ? 16 * p : 0));
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) {
                const float4 c = __ldg(c4 + jj), sn = __ldg(s4 + jj);
                const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int j = jj * 4 + e;
                  const float x1 = lo[j], x2 = hi[j];
                  lo[j] = x1 * cc[e] - x2 * ss[e];
                  hi[j] = x2 * cc[e] + x1 * ss[e];
                }
              }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint4 o;
              o.x = pack_bf2(lo[h * 8 + 0], lo[h * 8 + 1]); o.y = pack_bf2(lo[h * 8 + 2], lo[h * 8 + 3]);
              o.z = pack_bf2(lo[h * 8 + 4], lo[h * 8 + 5]); o.w = pack_bf2(lo[h * 8 + 6], lo[h * 8 + 7]);
              st_shared_v4(row_addr + ((uint32_t)(((lo_col >> 3) + h) ^ sw) << 4), o);
              o.x = pack_bf2(hi[h * 8 + 0], hi[h * 8 + 1]); o.y = pack_bf2(hi[h * 8 + 2], hi[h * 8 + 3]);
              o.z = pack_bf2(hi[h * 8 + 4], hi[h * 8 + 5]); o.w = pack_bf2(hi[h * 8 + 6], hi[h * 8 + 7]);
              st_shared_v4(row_addr + ((uint32_t)(((hi_col >> 3) + h) ^ sw) << 4), o);
            }
          }
        } else {
          float ss_out = 0.f;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {              // two 32-column halves keep the register footprint low
            uint32_t r[32];
            tmem_ld32(taddr + hh * 32, r);
            if (hh == 1 && last_of_tile) release_acc(acc);
            float v[32];
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              v[k] = round_bf(__uint_as_float(r[k]) * rstd);                   // Linear output is bf16
              if (EPI == EPI_GELU) v[k] = gelu_tanh_f(v[k]);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint32_t addr = row_addr + ((uint32_t)((hh * 4 + c) ^ sw) << 4);
              if (RES) {
                const uint4 rr = ld_shared_v4(addr);
                const float2 a = unpack_bf2(rr.x), b = unpack_bf2(rr.y), cc = unpack_bf2(rr.z), d = unpack_bf2(rr.w);
                v[c * 8 + 0] += a.x; v[c * 8 + 1] += a.y; v[c * 8 + 2] += b.x; v[c * 8 + 3] += b.y;
                v[c * 8 + 4] += cc.x; v[c * 8 + 5] += cc.y; v[c * 8 + 6] += d.x; v[c * 8 + 7] += d.y;
#pragma unroll
                for (int k = 0; k < 8; ++k) ss_out += v[c * 8 + k] * v[c * 8 + k];   // statistics of the fp32 sums (pre-rounding)
              }
              uint4 o;
              o.x = pack_bf2(v[c * 8 + 0], v[c * 8 + 1]); o.y = pack_bf2(v[c * 8 + 2], v[c * 8 + 3]);
              o.z = pack_bf2(v[c * 8 + 4], v[c * 8 + 5]); o.w = pack_bf2(v[c * 8 + 6], v[c * 8 + 7]);
              st_shared_v4(addr, o);
            }
          }
          if (RES && norm.ss_out != nullptr && m0 + row_in_tile < M && c0 < N)
            norm.ss_out[(m0 + row_in_tile) * (long long)(N / SLAB_COLS) + c0 / SLAB_COLS] = ss_out;
        }
        fence_async_smem();
      }
      if (!epi_barrier_and(ok, 1 + gidx)) break;        // uniform over the group's 128 threads
      if (issuer && c0 < N && m0 < M) {
        tma_store_2d(&map_c, slab, c0, (int)m0);
        bulk_commit();
      }
    }
    if (issuer) bulk_wait_all();
  }

  // ---------------- teardown ----------------
  if (*verr != 0) __nanosleep(1000000);  // error path: let in-flight bulk copies land before the CTA retires
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA retires (or frees tensor memory) while the other may still signal or read it
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, cfg::TMEM_COLS);
    else tmem_dealloc(tmem_base, cfg::TMEM_COLS);
  }
  if (counters && blockIdx.x == 0 && threadIdx.x == 0) counters[6] = globaltimer_ns();   // CTA 0 done
}

template <int BN, int EPI, bool PAIR>
phx_status launch_t(const GemmPlan& p, const GemmRope& rope, const GemmNorm& norm, int64_t M, int* err_flag, int num_sms,
                    cudaStream_t stream, std::string& err) {
  // the residual epilogues are fed by TMA prefetch and keep up with two groups; the others (RoPE, GELU, norm
  // scaling) are bound by the latency of each thread's instruction stream and get four groups where a pair's
  // smaller stages leave room for the slab buffers
  constexpr int NG = (PAIR && EPI != EPI_RESIDUAL) ? 4 : 2;
  using cfg = Cfg<BN, PAIR, NG>;
  auto kern = gemm_tcgen05_kernel<BN, EPI, PAIR, NG>;
  static bool attr_set = false;
  static int max_pairs = 0;
  cudaLaunchConfig_t lc;
  memset(&lc, 0, sizeof(lc));
  cudaLaunchAttribute attr[2];
  lc.blockDim = dim3(gemm_threads(NG));
  lc.dynamicSmemBytes = cfg::SMEM_BYTES;
  lc.stream = stream;
  lc.attrs = attr; lc.numAttrs = 0;
  if (PAIR) {
    attr[lc.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[lc.numAttrs].val.clusterDim.x = 2; attr[lc.numAttrs].val.clusterDim.y = 1; attr[lc.numAttrs].val.clusterDim.z = 1;
    lc.numAttrs++;
  }
  const int attrs_for_query = lc.numAttrs;
  // the kernel's set-up may overlap the tail of the kernel in front of it (it waits before it reads global data);
  // PHX_PDL=0 keeps plain stream order
  static const bool pdl = !(getenv("PHX_PDL") && getenv("PHX_PDL")[0] == '0');
  if (pdl) {
    attr[lc.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[lc.numAttrs].val.programmaticStreamSerializationAllowed = 1;
    lc.numAttrs++;
  }
  if (!attr_set) {
    PHX_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES), err);
    if (PAIR) {   // how many CTA pairs the device can hold at once (pairs need two SMs of one cluster-capable group)
      lc.gridDim = dim3(2 * (num_sms / 2));
      int n = 0;
      const int all_attrs = lc.numAttrs;
      lc.numAttrs = attrs_for_query;   // the occupancy query takes the cluster shape only
      PHX_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &lc), err);
      lc.numAttrs = all_attrs;
      max_pairs = n < num_sms / 2 ? n : num_sms / 2;
      if (max_pairs <= 0) { err = "gemm: the device cannot hold a CTA pair of this kernel"; return PHX_E_CUDA; }
    }
    attr_set = true;
  }
  constexpr int TILE_M = PAIR ? 2 * BM : BM;
  const long long tiles = ((M + TILE_M - 1) / TILE_M) * ((p.N + BN - 1) / BN);
  const int slots = PAIR ? max_pairs : num_sms;
  const int units = (int)(tiles < slots ? tiles : slots);
  if (units <= 0) return PHX_OK;
  lc.gridDim = dim3(PAIR ? 2 * units : units);
  const CUtensorMap& mr = (EPI == EPI_RESIDUAL) ? p.map_r : p.map_c;
  long long Mll = M;
  int N = p.N, K = p.K;
  unsigned long long* counters = p.counters;
  PHX_CUDA_TRY(cudaLaunchKernelEx(&lc, kern, p.map_a, p.map_b, p.map_c, mr, rope, norm, Mll, N, K, err_flag, counters), err);
  return PHX_OK;
}

template <int BN, bool PAIR>
phx_status launch_e(const GemmPlan& p, int epilogue, const GemmRope& rp, const GemmNorm& nm, int64_t M, int* err_flag,
                    int num_sms, cudaStream_t stream, std::string& err) {
  switch (epilogue) {
    case EPI_STORE: return launch_t<BN, EPI_STORE, PAIR>(p, rp, nm, M, err_flag, num_sms, stream, err);
    case EPI_RESIDUAL: return launch_t<BN, EPI_RESIDUAL, PAIR>(p, rp, nm, M, err_flag, num_sms, stream, err);
    case EPI_GELU: return launch_t<BN, EPI_GELU, PAIR>(p, rp, nm, M, err_flag, num_sms, stream, err);
    case EPI_ROPE: return launch_t<BN, EPI_ROPE, PAIR>(p, rp, nm, M, err_flag, num_sms, stream, err);
  }
  err = "gemm: unknown epilogue";
  return PHX_E_ARG;
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
                            bool narrow_tiles, std::string& err, int pair) {
  if (N % 8 != 0 || K % 8 != 0 || N <= 0 || K <= 0 || rows_max <= 0) {
    err = "gemm: N and K must be positive multiples of 8";
    return PHX_E_ARG;
  }
  plan->A = A; plan->Wt = Wt; plan->rows_max = rows_max; plan->a_rows = rows_max; plan->N = N; plan->K = K;
  // 128-wide tiles leave room for six output slabs: deep residual prefetch for the HBM-bound short-K GEMMs
  { const char* t = getenv("PHX_GEMM_TILES");   // diagnostics: wide | narrow overrides the caller's choice
    if (t && strcmp(t, "wide") == 0) narrow_tiles = false;
    if (t && strcmp(t, "narrow") == 0) narrow_tiles = true; }
  // CTA pairs by default; PHX_GEMM=cta1 keeps every CTA on its own tile (for comparison)
  const char* mode = getenv("PHX_GEMM");
  plan->pair = pair >= 0 ? (pair != 0) : !(mode && strcmp(mode, "cta1") == 0);
  // a pair fills 128 + BN/2 operand rows per CTA and k-step: the wide tile is the cheaper one per FLOP there
  // (out-projection, N = K = 512: 0.100 ms wide against 0.146 ms narrow)
  if (plan->pair && !(getenv("PHX_GEMM_TILES") && strcmp(getenv("PHX_GEMM_TILES"), "narrow") == 0)) narrow_tiles = false;
  plan->BN = (N % 256 == 0 && !narrow_tiles) ? 256 : 128;
  phx_status s = make_map(&plan->map_a, A, rows_max, K, BM, err);
  if (s != PHX_OK) return s;
  s = make_map(&plan->map_b, Wt, N, K, plan->pair ? plan->BN / 2 : plan->BN, err);
  if (s != PHX_OK) return s;
  if (plan->BN == 256) {   // small calls (a single request) run 128-column tiles: twice the CTAs, half the work per tile
    s = make_map(&plan->map_b_narrow, Wt, N, K, plan->pair ? 64 : 128, err);
    if (s != PHX_OK) return s;
    plan->has_narrow = true;
  }
  plan->ready = true;
  return PHX_OK;
}

phx_status gemm_launch(GemmPlan& p, const bf16* A, bf16* C, const bf16* R, int64_t M, int epilogue, const GemmRope* rope,
                       const GemmNorm* norm, int* err_flag, int num_sms, cudaStream_t stream, std::string& err) {
  if (!p.ready || M > p.rows_max) { err = "gemm: plan not ready or M exceeds plan rows"; return PHX_E_ARG; }
  if (epilogue == EPI_RESIDUAL && R == nullptr) { err = "gemm: residual epilogue needs R"; return PHX_E_ARG; }
  GemmRope rp;
  memset(&rp, 0, sizeof(rp));
  GemmNorm nm;
  memset(&nm, 0, sizeof(nm));
  if (norm) nm = *norm;
  if (nm.ss_out && (epilogue != EPI_RESIDUAL || p.N % SLAB_COLS != 0)) { err = "gemm: row statistics are produced by the residual epilogue only"; return PHX_E_ARG; }
  if (A != p.A || (p.a_rows != M && p.a_rows != p.rows_max)) {
    // the activation buffer moved (double-buffered residual stream, or a block of rows inside it): re-encode its
    // map over exactly the M rows of this call, so that no tile reads past them
    phx_status s = make_map(&p.map_a, A, M, p.K, BM, err);
    if (s != PHX_OK) return s;
    p.A = A; p.a_rows = M;
  }
  if (epilogue == EPI_ROPE) {
    if (!rope || (rope->dh != 32 && rope->dh != 64) || rope->T <= 0 || p.N % rope->dh != 0) {
      err = "gemm: the RoPE epilogue needs head dim 32 or 64";
      return PHX_E_ARG;
    }
    rp = *rope;
  }
  // output / residual maps are [M, N] with 128 x 64 boxes; rows past M are clipped by the TMA unit
  if (p.c_ptr != C || p.c_rows != M) {
    phx_status s = make_map(&p.map_c, C, M, p.N, BM, err);
    if (s != PHX_OK) return s;
    p.c_ptr = C; p.c_rows = M;
  }
  if (epilogue == EPI_RESIDUAL && (p.r_ptr != R || p.r_rows != M)) {
    phx_status s = make_map(&p.map_r, R, M, p.N, BM, err);
    if (s != PHX_OK) return s;
    p.r_ptr = R; p.r_rows = M;
  }
  if (p.BN == 256) {
    // latency regime: when even the 128-column tiles leave SMs idle, take them - the call's time is one tile's time
    const long long rows_per_tile = p.pair ? 2 * BM : BM;
    const long long narrow_tiles = ((M + rows_per_tile - 1) / rows_per_tile) * ((p.N + 127) / 128);
    const long long slots = p.pair ? num_sms / 2 : num_sms;
    static const bool allow = !(getenv("PHX_GEMM_TILES") && strcmp(getenv("PHX_GEMM_TILES"), "wide") == 0);
    if (allow && p.has_narrow && narrow_tiles <= slots) {
      dispatch_note(p.pair ? DK_GEMM_PAIR128 : DK_GEMM_CTA128);
      GemmPlan q = p;
      q.map_b = p.map_b_narrow; q.BN = 128;
      return q.pair ? launch_e<128, true>(q, epilogue, rp, nm, M, err_flag, num_sms, stream, err)
                    : launch_e<128, false>(q, epilogue, rp, nm, M, err_flag, num_sms, stream, err);
    }
    dispatch_note(p.pair ? DK_GEMM_PAIR256 : DK_GEMM_CTA256);
    return p.pair ? launch_e<256, true>(p, epilogue, rp, nm, M, err_flag, num_sms, stream, err)
                  : launch_e<256, false>(p, epilogue, rp, nm, M, err_flag, num_sms, stream, err);
  }
  dispatch_note(p.pair ? DK_GEMM_PAIR128 : DK_GEMM_CTA128);
  return p.pair ? launch_e<128, true>(p, epilogue, rp, nm, M, err_flag, num_sms, stream, err)
                : launch_e<128, false>(p, epilogue, rp, nm, M, err_flag, num_sms, stream, err);
}

namespace {
__global__ void wait_selftest_kernel(int* err_flag) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t b = smem_u32(&bar);
  mbar_init(b, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  mbar_wait(b, 0, err_flag);   // nothing arrives: returns false once the limit has passed
}
}  // namespace

phx_status wait_selftest_launch(int* err_flag, cudaStream_t stream, std::string& err) {
  wait_selftest_kernel<<<1, 1, 0, stream>>>(err_flag);
  PHX_CUDA_TRY(cudaGetLastError(), err);
  return PHX_OK;
}

phx_status gemm_simt_launch(const bf16* A, const bf16* Wt, bf16* C, const bf16* R, int64_t M, int N, int K,
                            int epilogue, cudaStream_t stream, std::string& err) {
  dispatch_note(DK_GEMM_SIMT);
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
