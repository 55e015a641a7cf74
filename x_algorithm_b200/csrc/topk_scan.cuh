// Interface of the tcgen05 corpus scan (topk_scan_sm100.cu) used by the top-k driver (topk.cu).
#pragma once

#include "common.cuh"

namespace phx {

struct TcScanArgs {
  long long rows;            // corpus rows of this shard
  long long row_offset;      // global id of local row 0
  int dim, B;                // embedding dim (64 or 128), live queries (<= 256)
  int stride;                // sample pass: tiles 0, stride, 2*stride, ...
  float* gmax;               // sample pass out: [B][n_groups] maxima of 32-row groups
  long long n_groups;        // sampled tiles * 4
  const float* pivot;        // collect pass in: [B]
  unsigned long long* surv;  // collect pass out: [B][cap] keys ordered(score) << 32 | ~global_row
  int* counts;               // [B]
  int cap;
  // optional eligibility of the shard's rows: bit (r & 31) of mask[r >> 5] for shard-local row r = mask_row0 + row;
  // a row whose bit is clear is skipped like a row past the end.  null = every row is eligible
  const unsigned int* mask = nullptr;
  long long mask_row0 = 0;
};

__device__ __forceinline__ bool row_eligible(const unsigned int* mask, long long mask_row0, long long row) {
  if (!mask) return true;
  const long long r = mask_row0 + row;
  return (mask[r >> 5] >> (r & 31)) & 1u;
}

bool tc_scan_supported(int dim);
phx_status tc_scan_make_maps(CUtensorMap* map_corpus, CUtensorMap* map_users, const bf16* corpus, long long rows, int dim,
                             const bf16* users_bf, std::string& err);
// mode 0 = sample pass (group maxima), 1 = collect pass (survivors)
phx_status tc_scan_launch(const CUtensorMap& map_corpus, const CUtensorMap& map_users, const TcScanArgs& a, int mode,
                          int num_sms, int* err_flag, cudaStream_t stream, std::string& err);

}  // namespace phx
