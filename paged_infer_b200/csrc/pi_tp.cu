// Tensor parallelism plumbing: one process per GPU, NCCL over NVLink/NVSwitch.
// Column-split q/k/v/gate/up need no exchange; row-split o/down are followed by
// one all-reduce of the [B x hidden] partial sums; the vocab-split LM head by one
// all-gather.  NCCL is bound at run time (dlopen) so that single-GPU users do
// not need it.  The reference has no multi-device code; nothing is replaced.
#include <dlfcn.h>
#include <nccl.h>

#include "pi_common.cuh"

namespace {
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string error;
};

NcclApi* nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return &api;
  tried = true;
  api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!api.handle) {
    api.error = std::string("cannot load libnccl.so.2: ") + dlerror();
    return &api;
  }
#define PI_SYM(field, name)                                                  \
  api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, name)); \
  if (!api.field) api.error = std::string("libnccl lacks ") + name;
  PI_SYM(GetUniqueId, "ncclGetUniqueId")
  PI_SYM(CommInitRank, "ncclCommInitRank")
  PI_SYM(CommDestroy, "ncclCommDestroy")
  PI_SYM(AllReduce, "ncclAllReduce")
  PI_SYM(AllGather, "ncclAllGather")
  PI_SYM(GetErrorString, "ncclGetErrorString")
#undef PI_SYM
  return &api;
}
}  // namespace

#define PI_NCCL(ctx, expr)                                                                          \
  do {                                                                                              \
    ncclResult_t _r = (expr);                                                                       \
    if (_r != ncclSuccess)                                                                          \
      return pi_fail((ctx), PI_ERR_NCCL, "%s failed: %s", #expr, nccl()->GetErrorString(_r));       \
  } while (0)

extern "C" pi_status pi_nccl_unique_id(void* out_128_bytes) {
  if (!out_128_bytes) return pi_fail(nullptr, PI_ERR_INVALID_ARG, "null pointer");
  NcclApi* n = nccl();
  if (!n->error.empty()) return pi_fail(nullptr, PI_ERR_NCCL, "%s", n->error.c_str());
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  ncclResult_t r = n->GetUniqueId(&id);
  if (r != ncclSuccess) return pi_fail(nullptr, PI_ERR_NCCL, "ncclGetUniqueId: %s", n->GetErrorString(r));
  memcpy(out_128_bytes, &id, sizeof(id));
  return PI_OK;
}

pi_status pi_tp_init(pi_ctx* ctx, const void* unique_id) {
  NcclApi* n = nccl();
  if (!n->error.empty()) return pi_fail(ctx, PI_ERR_NCCL, "%s", n->error.c_str());
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  ncclComm_t comm = nullptr;
  PI_NCCL(ctx, n->CommInitRank(&comm, ctx->tp, id, ctx->rank));
  ctx->nccl_comm = comm;
  return PI_OK;
}

void pi_tp_destroy(pi_ctx* ctx) {
  if (ctx->nccl_comm) {
    nccl()->CommDestroy(static_cast<ncclComm_t>(ctx->nccl_comm));
    ctx->nccl_comm = nullptr;
  }
}

pi_status pi_tp_all_reduce_sum(pi_ctx* ctx, float* buf, size_t n) {
  if (ctx->tp == 1 || n == 0) return PI_OK;
  pi_prof_scope prof(ctx, PI_PROF_COLLECTIVE);
  PI_NCCL(ctx, nccl()->AllReduce(buf, buf, n, ncclFloat32, ncclSum, static_cast<ncclComm_t>(ctx->nccl_comm), ctx->stream));
  return PI_OK;
}

pi_status pi_tp_all_gather(pi_ctx* ctx, const void* send, void* recv, size_t bytes_per_rank) {
  if (ctx->tp == 1) {
    PI_CUDA(ctx, cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
    return PI_OK;
  }
  PI_NCCL(ctx, nccl()->AllGather(send, recv, bytes_per_rank, ncclInt8, static_cast<ncclComm_t>(ctx->nccl_comm), ctx->stream));
  return PI_OK;
}
