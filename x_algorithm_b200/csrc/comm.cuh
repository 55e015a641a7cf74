// The library's own communicator (include/phoenix_b200.h, phx_comm_*): one NCCL communicator per rank, created from
// a unique id the host ships between its processes, plus the small collectives the sharded paths are built from.
// NCCL is bound at run time (dlopen of libnccl.so.2: the copy a host process has already loaded, else the system's), so
// single-GPU users of the library need no NCCL at all.  The reference's row-sharded embedding owns its communicator the
// same way (phoenix/xrex/cuda/row_emb/src/row_emb_comm.cc:283-345).
#pragma once

#include <nccl.h>

#include <functional>
#include <string>
#include <vector>

#include "common.cuh"

namespace phx {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
};
// null when libnccl cannot be loaded (err says why)
const NcclApi* nccl_api(std::string& err);

}  // namespace phx

struct phx_comm {
  int rank = 0, world = 1, device = 0;
  ncclComm_t comm = nullptr;
  const phx::NcclApi* api = nullptr;
  std::string err;
  cudaStream_t side[4] = {nullptr, nullptr, nullptr, nullptr};   // copy-engine transfers beside the caller's stream
  cudaEvent_t ev_fork = nullptr, ev_join[4] = {nullptr, nullptr, nullptr, nullptr};
  int* fence = nullptr;                                          // one int for ordering all-reduces
  // work spaces of the sharded paths, owned here so that they die with the communicator
  void* gather_ws = nullptr;
  std::function<void(void*, int)> gather_ws_free;   // (work space, step): 0 unmap peer memory, 1 free own memory
  unsigned long long* keys_local = nullptr;   // retrieval: this shard's list [B*k] + the lists of all ranks [W*B*k]
  unsigned long long* keys_all = nullptr;
  int* status_all = nullptr;                  // [W + 1]: every rank's scan status, then their OR
  int* status_host = nullptr;                 // pinned
  size_t keys_cap = 0;
};

namespace phx {
// NCCL call -> status; on failure comm->err names the call
phx_status comm_check(phx_comm* c, ncclResult_t r, const char* what);
}  // namespace phx
