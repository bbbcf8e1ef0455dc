// NCCL communicator of a context: the one collective of this library is an all-gather of device buffers on the
// context's stream (hidden rows and per-row acceptance statistics of the vocabulary-sharded LM head).
//
// NCCL is bound at run time (dlopen of libnccl.so.2): a process that already loaded it -- torch does -- shares
// that copy, a process without NCCL still loads this library and gets VN_ERR_NCCL from these entry points only.
// Peers' data always lands in this GPU's own memory before a kernel of this library reads it.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

struct vn_comm {
  vn_ctx* ctx = nullptr;
  ncclComm_t comm = nullptr;
  int world = 1, rank = 0;
};

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi& nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) return;
    api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
    api.AllGather = (decltype(api.AllGather))dlsym(api.handle, "ncclAllGather");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.GetErrorString;
  });
  return api;
}

int32_t nccl_fail(vn_ctx* ctx, const char* what, ncclResult_t r) {
  return vn_fail(ctx, VN_ERR_NCCL, "%s failed: %s", what, nccl_api().GetErrorString ? nccl_api().GetErrorString(r) : "?");
}

}  // namespace

extern "C" {

int32_t vn_comm_unique_id(uint8_t* out128) {
  if (!out128) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  NcclApi& api = nccl_api();
  if (!api.ok) return vn_fail(nullptr, VN_ERR_NCCL, "libnccl.so.2 could not be loaded");
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  ncclResult_t r = api.GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(nullptr, "ncclGetUniqueId", r);
  memcpy(out128, &id, 128);
  return VN_OK;
}

int32_t vn_comm_create(vn_ctx* ctx, const uint8_t* unique_id128, int32_t world, int32_t rank, vn_comm** out) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, unique_id128 && out && world >= 1 && rank >= 0 && rank < world, "bad arguments");
  *out = nullptr;
  NcclApi& api = nccl_api();
  if (!api.ok) return vn_fail(ctx, VN_ERR_NCCL, "libnccl.so.2 could not be loaded");
  ncclUniqueId id;
  memcpy(&id, unique_id128, 128);
  vn_comm* c = new vn_comm();
  c->ctx = ctx; c->world = world; c->rank = rank;
  ncclResult_t r = api.CommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) { delete c; return nccl_fail(ctx, "ncclCommInitRank", r); }
  *out = c;
  return VN_OK;
}

int32_t vn_comm_destroy(vn_comm* c) {
  if (!c) return VN_OK;
  cudaSetDevice(c->ctx->device);
  cudaStreamSynchronize(c->ctx->stream);
  if (c->comm && nccl_api().ok) nccl_api().CommDestroy(c->comm);
  delete c;
  return VN_OK;
}

int32_t vn_comm_info(vn_comm* c, int32_t* world, int32_t* rank) {
  if (!c) return vn_fail(nullptr, VN_ERR_INVALID, "null communicator");
  if (world) *world = c->world;
  if (rank) *rank = c->rank;
  return VN_OK;
}

int32_t vn_all_gather(vn_comm* c, const void* send_dev, void* recv_dev, size_t bytes_per_rank) {
  if (!c) return vn_fail(nullptr, VN_ERR_INVALID, "null communicator");
  vn_ctx* ctx = c->ctx;
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, send_dev && recv_dev, "null buffer");
  if (bytes_per_rank == 0) return VN_OK;
  ncclResult_t r = nccl_api().AllGather(send_dev, recv_dev, bytes_per_rank, ncclUint8, c->comm, ctx->stream);
  if (r != ncclSuccess) return nccl_fail(ctx, "ncclAllGather", r);
  return VN_OK;
}

}  // extern "C"

// used by the sharded acceptance (accept.cu): a missing communicator is a world of one
int32_t vn_comm_gather(vn_ctx* ctx, vn_comm* c, const void* send_dev, void* recv_dev, size_t bytes_per_rank, int* world,
                       int* rank) {
  if (world) *world = c ? c->world : 1;
  if (rank) *rank = c ? c->rank : 0;
  if (bytes_per_rank == 0) return VN_OK;
  if (!c || c->world == 1) {
    if (send_dev != recv_dev)
      VN_CUDA(ctx, cudaMemcpyAsync(recv_dev, send_dev, bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
    return VN_OK;
  }
  return vn_all_gather(c, send_dev, recv_dev, bytes_per_rank);
}
