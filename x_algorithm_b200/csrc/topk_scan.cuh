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
};

bool tc_scan_supported(int dim);
phx_status tc_scan_make_maps(CUtensorMap* map_corpus, CUtensorMap* map_users, const bf16* corpus, long long rows, int dim,
                             const bf16* users_bf, std::string& err);
// mode 0 = sample pass (group maxima), 1 = collect pass (survivors)
phx_status tc_scan_launch(const CUtensorMap& map_corpus, const CUtensorMap& map_users, const TcScanArgs& a, int mode,
                          int num_sms, int* err_flag, cudaStream_t stream, std::string& err);

}  // namespace phx
