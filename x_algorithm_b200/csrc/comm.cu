// phx_comm_*: the communicator the C ABI owns.  See comm.cuh.
#include <dlfcn.h>
#include <string.h>

#include <mutex>

#include "comm.cuh"

namespace phx {

const NcclApi* nccl_api(std::string& err) {
  static NcclApi api;
  static bool tried = false, ok = false;
  static std::string why;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  if (!tried) {
    tried = true;
    // a process that has NCCL loaded already (a framework's bundled copy) gets that copy: same soname
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { why = std::string("NCCL is not available: ") + dlerror(); }
    else {
      bool all = true;
      auto bind = [&](auto& fn, const char* name) {
        fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(dlsym(h, name));
        if (!fn) { all = false; why = std::string("libnccl lacks ") + name; }
      };
      bind(api.GetUniqueId, "ncclGetUniqueId"); bind(api.CommInitRank, "ncclCommInitRank");
      bind(api.CommDestroy, "ncclCommDestroy"); bind(api.CommAbort, "ncclCommAbort");
      bind(api.AllGather, "ncclAllGather"); bind(api.AllReduce, "ncclAllReduce");
      bind(api.Send, "ncclSend"); bind(api.Recv, "ncclRecv");
      bind(api.GroupStart, "ncclGroupStart"); bind(api.GroupEnd, "ncclGroupEnd");
      bind(api.GetErrorString, "ncclGetErrorString"); bind(api.GetVersion, "ncclGetVersion");
      ok = all;
    }
  }
  if (!ok) { err = why; return nullptr; }
  return &api;
}

phx_status comm_check(phx_comm* c, ncclResult_t r, const char* what) {
  if (r == ncclSuccess) return PHX_OK;
  c->err = std::string(what) + ": " + (c->api && c->api->GetErrorString ? c->api->GetErrorString(r) : "NCCL error");
  return PHX_E_NCCL;
}

}  // namespace phx

using namespace phx;

extern "C" {

phx_status phx_comm_unique_id(uint8_t out[PHX_COMM_ID_BYTES]) {
  static_assert(sizeof(ncclUniqueId) == PHX_COMM_ID_BYTES, "unique id size");
  if (!out) { set_global_error("phx_comm_unique_id: null argument"); return PHX_E_ARG; }
  std::string err;
  const NcclApi* api = nccl_api(err);
  if (!api) { set_global_error(err); return PHX_E_NCCL; }
  ncclUniqueId id;
  const ncclResult_t r = api->GetUniqueId(&id);
  if (r != ncclSuccess) { set_global_error(std::string("ncclGetUniqueId: ") + api->GetErrorString(r)); return PHX_E_NCCL; }
  memcpy(out, &id, sizeof(id));
  return PHX_OK;
}

phx_status phx_comm_create(const uint8_t id_bytes[PHX_COMM_ID_BYTES], int32_t rank, int32_t world, int32_t device, phx_comm** out) {
  if (!id_bytes || !out || world < 1 || world > PHX_MAX_SHARDS || rank < 0 || rank >= world) {
    set_global_error("phx_comm_create: bad argument (1 <= world <= 16, 0 <= rank < world)");
    return PHX_E_ARG;
  }
  std::string err;
  const NcclApi* api = nccl_api(err);
  if (!api) { set_global_error(err); return PHX_E_NCCL; }
  if (cudaSetDevice(device) != cudaSuccess) { set_global_error("phx_comm_create: cudaSetDevice failed"); return PHX_E_CUDA; }
  phx_comm* c = new phx_comm();
  c->rank = rank; c->world = world; c->device = device; c->api = api;
  ncclUniqueId id;
  memcpy(&id, id_bytes, sizeof(id));
  const ncclResult_t r = api->CommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) {
    set_global_error(std::string("ncclCommInitRank: ") + api->GetErrorString(r));
    delete c;
    return PHX_E_NCCL;
  }
  bool ok = true;
  for (auto& s : c->side) ok = ok && cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming) == cudaSuccess;
  for (auto& e : c->ev_join) ok = ok && cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaMalloc(&c->fence, 64) == cudaSuccess && cudaMemset(c->fence, 0, 64) == cudaSuccess;
  ok = ok && cudaMalloc(&c->status_all, (PHX_MAX_SHARDS + 2) * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMallocHost(&c->status_host, (PHX_MAX_SHARDS + 2) * sizeof(int)) == cudaSuccess;
  if (!ok) { set_global_error("phx_comm_create: CUDA resources"); phx_comm_destroy(c); return PHX_E_CUDA; }
  *out = c;
  return PHX_OK;
}

void phx_comm_destroy(phx_comm* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  if (c->gather_ws && c->gather_ws_free) {
    // memory that other ranks have mapped is freed only after every rank has unmapped it (destroy is collective)
    c->gather_ws_free(c->gather_ws, 0);
    if (c->comm && c->world > 1 && c->api->AllReduce(c->fence, c->fence, 1, ncclInt32, ncclSum, c->comm, nullptr) == ncclSuccess)
      cudaStreamSynchronize(nullptr);
    c->gather_ws_free(c->gather_ws, 1);
  }
  if (c->keys_local) cudaFree(c->keys_local);
  if (c->keys_all) cudaFree(c->keys_all);
  if (c->status_all) cudaFree(c->status_all);
  if (c->status_host) cudaFreeHost(c->status_host);
  if (c->fence) cudaFree(c->fence);
  for (auto s : c->side) if (s) cudaStreamDestroy(s);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  for (auto e : c->ev_join) if (e) cudaEventDestroy(e);
  if (c->comm && c->api) c->api->CommDestroy(c->comm);
  delete c;
}

const char* phx_comm_last_error(const phx_comm* c) { return c ? c->err.c_str() : phx_global_error(); }

phx_status phx_comm_info(const phx_comm* c, int32_t* rank, int32_t* world, int32_t* nccl_version) {
  if (!c) return PHX_E_ARG;
  if (rank) *rank = c->rank;
  if (world) *world = c->world;
  if (nccl_version) { int v = 0; c->api->GetVersion(&v); *nccl_version = v; }
  return PHX_OK;
}

// Every rank waits here until all ranks have arrived (an all-reduce of one word on `stream`, then a stream sync).
phx_status phx_comm_barrier(phx_comm* c, void* stream) {
  if (!c) return PHX_E_ARG;
  cudaSetDevice(c->device);
  cudaStream_t st = (cudaStream_t)stream;
  phx_status s = comm_check(c, c->api->AllReduce(c->fence, c->fence, 1, ncclInt32, ncclSum, c->comm, st), "ncclAllReduce (barrier)");
  if (s) return s;
  PHX_CUDA_TRY(cudaStreamSynchronize(st), c->err);
  return PHX_OK;
}

}  // extern "C"
