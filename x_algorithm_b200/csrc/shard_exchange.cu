// Row-sharded embedding table, exchange by all-to-all: the device-side steps around the two collectives of the
// reference's id / row exchange (phoenix/xrex/cuda/row_emb/src/row_emb_comm.cc:655-743: ids to their owners, the
// owner-side gather, rows back to the requesters; combine by sum as recsys_embedding.py:282-331).
//
//   requester:  hash ids -> unified-table rows (phx_hash_ids_device)
//               phx_shard_bucket:       group the row requests by owning rank (counting sort over `world` buckets),
//                                       remember where each request went
//   collective: counts, then the local row numbers, to their owners        (NCCL all-to-all, issued by the host side)
//   owner:      phx_shard_gather_rows:  copy the requested rows of the local shard into one send block
//   collective: the rows back to the requesters                            (NCCL all-to-all)
//   requester:  phx_shard_sum_rows:     per id, the fp32 sum of its rows in hash-slot order, one rounding to bf16
//
// The sum order is by hash slot and does not depend on how requests were grouped or on the number of ranks, so the
// result is bit-identical to the single-table gather-sum kernel.  Every function launches on the stream it is
// given (the host side passes the stream its collectives run on) and allocates nothing.
#include <string.h>

#include <string>

#include "common.cuh"

namespace phx {
namespace {

constexpr int SX_THREADS = 256;
constexpr int SX_PER_THREAD = 8;
constexpr int SX_MAX_WORLD = 64;

// n_dev (optional): the request count lives on the device (the number of distinct rows a dedup pass found); n is then
// its upper bound, which sizes the grid
__global__ void __launch_bounds__(SX_THREADS) sx_count_kernel(const int* __restrict__ rows, long long n, const int* __restrict__ n_dev,
                                                              long long rows_per_shard, int world, int* __restrict__ counts) {
  __shared__ int hist[SX_MAX_WORLD];
  if (n_dev && *n_dev < n) n = *n_dev;
  if (threadIdx.x < world) hist[threadIdx.x] = 0;
  __syncthreads();
  const long long base = (long long)blockIdx.x * SX_THREADS * SX_PER_THREAD;
#pragma unroll
  for (int k = 0; k < SX_PER_THREAD; ++k) {
    const long long i = base + k * SX_THREADS + threadIdx.x;
    if (i < n) atomicAdd(&hist[(int)(rows[i] / rows_per_shard)], 1);
  }
  __syncthreads();
  if (threadIdx.x < world && hist[threadIdx.x]) atomicAdd(&counts[threadIdx.x], hist[threadIdx.x]);
}

// cursor[o] = first slot of owner o's bucket (exclusive scan of the counts)
__global__ void sx_scan_kernel(const int* __restrict__ counts, int world, int* __restrict__ cursor) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int run = 0;
    for (int o = 0; o < world; ++o) { cursor[o] = run; run += counts[o]; }
  }
}

// Each block reserves a range in every bucket for its own requests with one global atomic per owner, then places
// them with shared-memory atomics.  The order inside a bucket is arbitrary; `pos` records it.
__global__ void __launch_bounds__(SX_THREADS) sx_scatter_kernel(const int* __restrict__ rows, long long n, const int* __restrict__ n_dev,
                                                                long long rows_per_shard, int world, int* __restrict__ cursor,
                                                                int* __restrict__ send_rows, int* __restrict__ pos) {
  __shared__ int hist[SX_MAX_WORLD];
  __shared__ int gbase[SX_MAX_WORLD];
  if (n_dev && *n_dev < n) n = *n_dev;
  if (threadIdx.x < world) hist[threadIdx.x] = 0;
  __syncthreads();
  const long long base = (long long)blockIdx.x * SX_THREADS * SX_PER_THREAD;
  int owner[SX_PER_THREAD], local[SX_PER_THREAD], slot[SX_PER_THREAD];
#pragma unroll
  for (int k = 0; k < SX_PER_THREAD; ++k) {
    const long long i = base + k * SX_THREADS + threadIdx.x;
    owner[k] = -1;
    if (i < n) {
      const int r = rows[i];
      owner[k] = (int)(r / rows_per_shard);
      local[k] = (int)(r - owner[k] * rows_per_shard);
      slot[k] = atomicAdd(&hist[owner[k]], 1);
    }
  }
  __syncthreads();
  if (threadIdx.x < world) gbase[threadIdx.x] = hist[threadIdx.x] ? atomicAdd(&cursor[threadIdx.x], hist[threadIdx.x]) : 0;
  __syncthreads();
#pragma unroll
  for (int k = 0; k < SX_PER_THREAD; ++k) {
    if (owner[k] >= 0) {
      const long long i = base + k * SX_THREADS + threadIdx.x;
      const int p = gbase[owner[k]] + slot[k];
      send_rows[p] = local[k];
      pos[i] = p;
    }
  }
}

// one warp per requested row: 16 bytes per lane and step
__global__ void __launch_bounds__(256) sx_gather_rows_kernel(const bf16* __restrict__ shard, long long shard_rows,
                                                             const int* __restrict__ idx, long long m, int width,
                                                             bf16* __restrict__ out) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= m) return;
  long long r = idx[w];
  if (r < 0 || r >= shard_rows) r = 0;   // out of range -> row 0, like the reference gather (emb_table.rs:124-140)
  const uint4* src = reinterpret_cast<const uint4*>(shard + r * width);
  uint4* dst = reinterpret_cast<uint4*>(out + w * width);
  for (int c = lane; c < width / 8; c += 32) __stcs(dst + c, __ldg(src + c));
}

// one warp per id: rows at pos[i*H + h], h = 0..H-1, summed in that order in fp32, rounded once
__global__ void __launch_bounds__(256) sx_sum_rows_kernel(const bf16* __restrict__ rows, const int* __restrict__ pos, long long n,
                                                          int H, int width, bf16* __restrict__ out) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  int p[PHX_MAX_HASHES];
#pragma unroll
  for (int h = 0; h < PHX_MAX_HASHES; ++h) p[h] = (h < H) ? pos[i * H + h] : 0;
  for (int c = lane; c < width / 8; c += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int h = 0; h < PHX_MAX_HASHES; ++h) {
      if (h < H) {
        const uint4 u = __ldcs(reinterpret_cast<const uint4*>(rows + (long long)p[h] * width) + c);
        const float2 a = unpack_bf2(u.x), b = unpack_bf2(u.y), cc = unpack_bf2(u.z), d = unpack_bf2(u.w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
        acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
      }
    }
    uint4 o;
    o.x = pack_bf2(acc[0], acc[1]); o.y = pack_bf2(acc[2], acc[3]); o.z = pack_bf2(acc[4], acc[5]); o.w = pack_bf2(acc[6], acc[7]);
    __stcs(reinterpret_cast<uint4*>(out + i * width) + c, o);
  }
}

// Owner side with the row transfer folded in: request j belongs to the requester r with seg[r] <= j < seg[r+1]; its row
// goes straight into that requester's landing buffer (a peer mapping, or local memory for r = this rank) at row
// j - seg[r] of the bucket the requester reserved for this owner.  One warp per row: a 512-byte row is one coalesced
// store of 32 x 16 bytes, which is what NVLink moves best; stores are posted, so the kernel does not wait on the link.
__global__ void __launch_bounds__(256) sx_gather_push_kernel(const bf16* __restrict__ shard, long long shard_rows,
                                                             const int* __restrict__ idx, const long long* __restrict__ seg,
                                                             const unsigned long long* __restrict__ dest, int world, int width) {
  __shared__ long long s_seg[SX_MAX_WORLD + 1];
  __shared__ unsigned long long s_dest[SX_MAX_WORLD];
  if (threadIdx.x <= world) s_seg[threadIdx.x] = seg[threadIdx.x];
  if (threadIdx.x < world) s_dest[threadIdx.x] = dest[threadIdx.x];
  __syncthreads();
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= s_seg[world]) return;
  int r = 0;
  while (r + 1 < world && w >= s_seg[r + 1]) ++r;
  long long row = idx[w];
  if (row < 0 || row >= shard_rows) row = 0;
  const uint4* src = reinterpret_cast<const uint4*>(shard + row * width);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(s_dest[r]) + (w - s_seg[r]) * width);
  for (int c = lane; c < width / 8; c += 32) dst[c] = __ldg(src + c);
}

// ---- duplicate requests ------------------------------------------------------------------------------------------------
// Zipf-distributed ids ask for the same rows again and again (three of four row reads of the single-GPU gather hit
// L2); only distinct rows need to cross NVLink.  An open-addressing table (64-bit entries: row + 1 in the low word, the
// row's index in the list of distinct rows in the high word; 0 = empty) finds them without sorting.
__device__ __forceinline__ uint32_t sx_mix(uint32_t x) {
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
  return x;
}

__global__ void __launch_bounds__(256) sx_dedup_insert_kernel(const int* __restrict__ rows, long long n, unsigned long long* table,
                                                              unsigned int mask, int* __restrict__ slot_of) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long key = (unsigned long long)((unsigned int)rows[i]) + 1ull;
  unsigned int s = sx_mix((unsigned int)key) & mask;
  for (;;) {
    const unsigned long long old = atomicCAS(&table[s], 0ull, key);
    if (old == 0ull || (old & 0xFFFFFFFFull) == key) break;   // claimed the slot, or the row is already there
    s = (s + 1) & mask;                                       // the table is at most half full: the probe ends
  }
  slot_of[i] = (int)s;
}

// every occupied slot gets the next index in the list of distinct rows (one global atomic per block)
__global__ void __launch_bounds__(256) sx_dedup_compact_kernel(unsigned long long* table, long long cap, int* __restrict__ urows,
                                                               int* __restrict__ nu) {
  __shared__ int s_cnt, s_base;
  if (threadIdx.x == 0) s_cnt = 0;
  __syncthreads();
  const long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  unsigned long long e = (s < cap) ? table[s] : 0ull;
  int my = -1;
  if (e != 0ull) my = atomicAdd(&s_cnt, 1);
  __syncthreads();
  if (threadIdx.x == 0) s_base = s_cnt ? atomicAdd(nu, s_cnt) : 0;
  __syncthreads();
  if (my >= 0) {
    const int u = s_base + my;
    urows[u] = (int)((e & 0xFFFFFFFFull) - 1ull);
    table[s] = (e & 0xFFFFFFFFull) | ((unsigned long long)(unsigned int)u << 32);
  }
}

// request i -> slot of its distinct row in the grouped order
__global__ void __launch_bounds__(256) sx_dedup_expand_kernel(const int* __restrict__ slot_of, const unsigned long long* __restrict__ table,
                                                              const int* __restrict__ upos, long long n, int* __restrict__ pos) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  pos[i] = upos[(int)(table[slot_of[i]] >> 32)];
}

phx_status fail_arg(const char* msg) { set_global_error(msg); return PHX_E_ARG; }
phx_status check_launch(const char* what) {
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) { set_global_error(std::string(what) + ": " + cudaGetErrorString(ce)); return PHX_E_CUDA; }
  return PHX_OK;
}

}  // namespace

phx_status shard_bucket_launch(const int* rows_dev, long long n_req, const int* n_dev, long long rows_per_shard, int world,
                               int* counts_dev, int* cursor_dev, int* send_rows_dev, int* pos_dev, cudaStream_t st) {
  if (!rows_dev || !counts_dev || !cursor_dev || !send_rows_dev || !pos_dev || n_req < 0 || rows_per_shard <= 0 || world < 1 ||
      world > SX_MAX_WORLD)
    return fail_arg("phx_shard_bucket: bad argument (world must be 1..64)");
  if (cudaMemsetAsync(counts_dev, 0, sizeof(int32_t) * world, st) != cudaSuccess) return check_launch("phx_shard_bucket");
  if (n_req > 0) {
    const unsigned blocks = (unsigned)((n_req + SX_THREADS * SX_PER_THREAD - 1) / (SX_THREADS * SX_PER_THREAD));
    sx_count_kernel<<<blocks, SX_THREADS, 0, st>>>(rows_dev, n_req, n_dev, rows_per_shard, world, counts_dev);
    sx_scan_kernel<<<1, 32, 0, st>>>(counts_dev, world, cursor_dev);
    sx_scatter_kernel<<<blocks, SX_THREADS, 0, st>>>(rows_dev, n_req, n_dev, rows_per_shard, world, cursor_dev, send_rows_dev, pos_dev);
  }
  return check_launch("phx_shard_bucket");
}

}  // namespace phx

using namespace phx;

extern "C" {

phx_status phx_shard_bucket(const int32_t* rows_dev, int64_t n_req, int64_t rows_per_shard, int32_t world, int32_t* counts_dev,
                            int32_t* cursor_dev, int32_t* send_rows_dev, int32_t* pos_dev, void* stream) {
  return shard_bucket_launch(rows_dev, n_req, nullptr, rows_per_shard, world, counts_dev, cursor_dev, send_rows_dev, pos_dev,
                             (cudaStream_t)stream);
}

phx_status phx_shard_gather_rows(const uint16_t* shard_dev, int64_t shard_rows, const int32_t* local_rows_dev, int64_t m,
                                 int32_t width, uint16_t* out_dev, void* stream) {
  if (!shard_dev || shard_rows <= 0 || m < 0 || width <= 0 || width % 8 != 0 || (m > 0 && (!local_rows_dev || !out_dev)))
    return fail_arg("phx_shard_gather_rows: bad argument (width must be a multiple of 8)");
  if (m == 0) return PHX_OK;
  sx_gather_rows_kernel<<<(unsigned)((m * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)shard_dev, shard_rows, local_rows_dev, m, width, (bf16*)out_dev);
  return check_launch("phx_shard_gather_rows");
}

phx_status phx_shard_sum_rows(const uint16_t* rows_dev, const int32_t* pos_dev, int64_t n, int32_t num_hashes, int32_t width,
                              uint16_t* out_dev, void* stream) {
  if (n < 0 || num_hashes < 1 || num_hashes > PHX_MAX_HASHES || width <= 0 || width % 8 != 0 ||
      (n > 0 && (!rows_dev || !pos_dev || !out_dev)))
    return fail_arg("phx_shard_sum_rows: bad argument");
  if (n == 0) return PHX_OK;
  sx_sum_rows_kernel<<<(unsigned)((n * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)rows_dev, pos_dev, n, num_hashes, width, (bf16*)out_dev);
  return check_launch("phx_shard_sum_rows");
}

phx_status phx_shard_gather_push(const uint16_t* shard_dev, int64_t shard_rows, const int32_t* local_rows_dev, int64_t m,
                                 const int64_t* seg_dev, const uint64_t* dest_dev, int32_t world, int32_t width, void* stream) {
  if (!shard_dev || shard_rows <= 0 || m < 0 || !seg_dev || !dest_dev || world < 1 || world > SX_MAX_WORLD || width <= 0 ||
      width % 8 != 0 || (m > 0 && !local_rows_dev))
    return fail_arg("phx_shard_gather_push: bad argument (world must be 1..64, width a multiple of 8)");
  if (m == 0) return PHX_OK;
  sx_gather_push_kernel<<<(unsigned)((m * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)shard_dev, shard_rows, local_rows_dev, (const long long*)seg_dev, (const unsigned long long*)dest_dev, world, width);
  return check_launch("phx_shard_gather_push");
}

phx_status phx_shard_dedup(const int32_t* rows_dev, int64_t n_req, uint64_t* table_dev, int64_t table_slots, int32_t* slot_dev,
                           int32_t* urows_dev, int32_t* nu_dev, void* stream) {
  if (n_req < 0 || !table_dev || !nu_dev || table_slots < 2 || (table_slots & (table_slots - 1)) != 0 || table_slots < 2 * n_req ||
      table_slots > (1ll << 31) || (n_req > 0 && (!rows_dev || !slot_dev || !urows_dev)))
    return fail_arg("phx_shard_dedup: bad argument (table_slots must be a power of two >= 2 * n_req)");
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(table_dev, 0, sizeof(uint64_t) * (size_t)table_slots, st) != cudaSuccess) return check_launch("phx_shard_dedup");
  if (cudaMemsetAsync(nu_dev, 0, sizeof(int32_t), st) != cudaSuccess) return check_launch("phx_shard_dedup");
  if (n_req > 0) {
    sx_dedup_insert_kernel<<<(unsigned)((n_req + 255) / 256), 256, 0, st>>>(rows_dev, n_req, (unsigned long long*)table_dev,
                                                                          (unsigned int)(table_slots - 1), slot_dev);
    sx_dedup_compact_kernel<<<(unsigned)((table_slots + 255) / 256), 256, 0, st>>>((unsigned long long*)table_dev, table_slots,
                                                                                  urows_dev, nu_dev);
  }
  return check_launch("phx_shard_dedup");
}

phx_status phx_shard_dedup_expand(const int32_t* slot_dev, const uint64_t* table_dev, const int32_t* upos_dev, int64_t n_req,
                                  int32_t* pos_dev, void* stream) {
  if (n_req < 0 || (n_req > 0 && (!slot_dev || !table_dev || !upos_dev || !pos_dev))) return fail_arg("phx_shard_dedup_expand: bad argument");
  if (n_req == 0) return PHX_OK;
  sx_dedup_expand_kernel<<<(unsigned)((n_req + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      slot_dev, (const unsigned long long*)table_dev, upos_dev, n_req, pos_dev);
  return check_launch("phx_shard_dedup_expand");
}

phx_status phx_copy_async(void* dst, const void* src, uint64_t bytes, void* stream) {
  if (bytes == 0) return PHX_OK;
  if (!dst || !src) return fail_arg("phx_copy_async: null pointer");
  cudaError_t ce = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, (cudaStream_t)stream);   // unified addressing: local or peer
  if (ce != cudaSuccess) { set_global_error(std::string("phx_copy_async: ") + cudaGetErrorString(ce)); return PHX_E_CUDA; }
  return PHX_OK;
}

phx_status phx_ipc_alloc(int32_t device, uint64_t bytes, void** ptr_out, uint8_t handle_out[PHX_IPC_HANDLE_BYTES]) {
  if (!ptr_out || !handle_out || bytes == 0) return fail_arg("phx_ipc_alloc: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == PHX_IPC_HANDLE_BYTES, "IPC handle size");
  if (cudaSetDevice(device) != cudaSuccess) return check_launch("phx_ipc_alloc");
  void* p = nullptr;
  cudaError_t ce = cudaMalloc(&p, bytes);
  if (ce != cudaSuccess) { set_global_error(std::string("phx_ipc_alloc: ") + cudaGetErrorString(ce)); return PHX_E_CUDA; }
  cudaIpcMemHandle_t h;
  ce = cudaIpcGetMemHandle(&h, p);
  if (ce != cudaSuccess) { cudaFree(p); set_global_error(std::string("phx_ipc_alloc: ") + cudaGetErrorString(ce)); return PHX_E_CUDA; }
  memcpy(handle_out, &h, sizeof(h));
  *ptr_out = p;
  return PHX_OK;
}

phx_status phx_ipc_open(int32_t device, const uint8_t handle[PHX_IPC_HANDLE_BYTES], void** ptr_out) {
  if (!handle || !ptr_out) return fail_arg("phx_ipc_open: bad argument");
  if (cudaSetDevice(device) != cudaSuccess) return check_launch("phx_ipc_open");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t ce = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (ce != cudaSuccess) { set_global_error(std::string("phx_ipc_open: ") + cudaGetErrorString(ce)); return PHX_E_CUDA; }
  *ptr_out = p;
  return PHX_OK;
}

phx_status phx_ipc_close(void* ptr) {
  if (!ptr) return PHX_OK;
  cudaError_t ce = cudaIpcCloseMemHandle(ptr);
  if (ce != cudaSuccess) { set_global_error(std::string("phx_ipc_close: ") + cudaGetErrorString(ce)); return PHX_E_CUDA; }
  return PHX_OK;
}

phx_status phx_ipc_free(void* ptr) {
  if (!ptr) return PHX_OK;
  cudaError_t ce = cudaFree(ptr);
  if (ce != cudaSuccess) { set_global_error(std::string("phx_ipc_free: ") + cudaGetErrorString(ce)); return PHX_E_CUDA; }
  return PHX_OK;
}

}  // extern "C"
