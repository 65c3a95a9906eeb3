// Tensor parallelism plumbing: one process per GPU, NCCL over NVLink/NVSwitch.
// Column-split q/k/v/gate/up need no exchange; row-split o/down are followed by
// one all-reduce of the [B x hidden] partial sums; the vocab-split LM head by one
// all-gather.  NCCL is bound at run time (dlopen) so that single-GPU users do
// not need it.  The reference has no multi-device code; nothing is replaced.
#include <dlfcn.h>

#include <algorithm>
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
  for (int r = 0; r < 8; ++r)
    if (ctx->peer.mapped[r]) {
      cudaIpcCloseMemHandle(ctx->peer.mapped[r]);
      ctx->peer.mapped[r] = nullptr;
    }
  if (ctx->peer.base) {
    cudaFree(ctx->peer.base);
    ctx->peer.base = nullptr;
  }
  ctx->peer.ready = false;
  if (ctx->nccl_comm) {
    nccl()->CommDestroy(static_cast<ncclComm_t>(ctx->nccl_comm));
    ctx->nccl_comm = nullptr;
  }
}

pi_status pi_tp_all_reduce_sum(pi_ctx* ctx, float* buf, size_t n) {
  if (ctx->tp == 1 || n == 0) return PI_OK;
  if (!ctx->nccl_comm) return pi_fail(ctx, PI_ERR_NCCL, "this tensor-parallel context has no NCCL communicator (created without a unique id) and its peer-memory exchange is not usable");
  pi_prof_scope prof(ctx, PI_PROF_COLLECTIVE);
  PI_NCCL(ctx, nccl()->AllReduce(buf, buf, n, ncclFloat32, ncclSum, static_cast<ncclComm_t>(ctx->nccl_comm), ctx->stream));
  return PI_OK;
}

pi_status pi_tp_all_gather(pi_ctx* ctx, const void* send, void* recv, size_t bytes_per_rank) {
  if (ctx->tp == 1) {
    PI_CUDA(ctx, cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
    return PI_OK;
  }
  if (!ctx->nccl_comm) return pi_fail(ctx, PI_ERR_NCCL, "this tensor-parallel context has no NCCL communicator (created without a unique id)");
  PI_NCCL(ctx, nccl()->AllGather(send, recv, bytes_per_rank, ncclInt8, static_cast<ncclComm_t>(ctx->nccl_comm), ctx->stream));
  return PI_OK;
}

// ---- peer-memory exchange ----------------------------------------------------------------------------------------
//
// Layout of every rank's allocation: [slot 0: tp regions of floats | slot 1: tp regions | flags[2][8] u64 | epoch[2] u64 |
// ticket[2] u32]; region r of a slot holds rank r's partial sums.  Two ways to fill it:
//   pull  a rank writes its partial sums into ITS OWN region of its own buffer, and the exchange kernel of every rank
//         reads region r from rank r's buffer (NVLink P2P loads);
//   push  the projection that produced the partial sums wrote them into its region of EVERY rank's buffer from its
//         epilogue (plain peer stores, posted while the rest of the projection is still computing), and the exchange
//         kernel reads all regions from its own memory.
// Two slots alternate between consecutive exchanges (o, down, o, ...).  A rank may overwrite slot s again (in its own
// or, pushing, in its peers' buffers) only after the exchange on slot 1-s, and that exchange cannot finish before every
// peer has started it, i.e. has finished reading slot s: no reader is ever overtaken.
namespace {
constexpr int kPeerSlots = 2;
constexpr int kPeerMaxTp = 8;

struct PeerReduceParams {
  float* x;                          // [rows][cols] residual stream, updated in place
  int rows, cols;
  int tp, rank, slot;
  const float* data[kPeerMaxTp];     // this slot of every rank
  unsigned long long* flags[kPeerMaxTp];   // flag arrays of every rank
  unsigned long long* epoch;         // local: epoch[slot]
  unsigned int* ticket;              // local: ticket[slot]
  int* err_flag;
  uint32_t spin_limit;               // polls (64 ns apart) before the wait for a peer gives up
  // optional: the new residual rows as bf16 planes (times a norm weight) + per-chunk sums of squares
  unsigned short* emit_base;
  size_t emit_plane_stride;
  const float* emit_norm;
  float* emit_sumsq;                 // [chunks per row][emit_sumsq_stride]
  size_t emit_sumsq_stride;
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {   // never from a stale L1 line
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

constexpr int kPeerChunk = 1024;     // floats of one row handled by one CTA pass (256 threads x float4)

// Every CTA reads the slot's epoch at its start and takes a ticket at its end; the CTA that draws the last ticket
// advances the epoch, so no CTA of this launch can read the advanced value (the grid is kept <= the SM count only to
// keep the waiting CTAs few).  A wait that runs out sets the context's error word and skips the add: the kernel
// always returns.
__global__ void __launch_bounds__(256) tp_peer_reduce_add_kernel(const PeerReduceParams p) {
  __shared__ int s_ok;
  __shared__ float s_red[8];
  pi_grid_dependency_wait();          // the partial sums of this rank come from the preceding kernel
  const unsigned long long e = *reinterpret_cast<volatile unsigned long long*>(p.epoch) + 1ull;
  if (blockIdx.x == 0 && threadIdx.x < p.tp && (int)threadIdx.x != p.rank) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + (size_t)p.slot * kPeerMaxTp + p.rank, e);   // "my slot is ready" on that peer
  }
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < p.tp && ok; ++r) {
      if (r == p.rank) continue;
      const unsigned long long* f = p.flags[p.rank] + (size_t)p.slot * kPeerMaxTp + r;
      uint32_t spin = 0;
      while (ld_acquire_sys(f) < e) {
        if (++spin >= p.spin_limit) {
          ok = 0;
          break;
        }
        __nanosleep(64);
      }
    }
    if (!ok && p.err_flag) atomicExch(p.err_flag, 9);
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    const int cpr = (p.cols + kPeerChunk - 1) / kPeerChunk;   // chunks per row
    for (int chunk = blockIdx.x; chunk < p.rows * cpr; chunk += gridDim.x) {
      const int row = chunk / cpr, seg = chunk - row * cpr;
      const int col = seg * kPeerChunk + threadIdx.x * 4;
      float sq = 0.f;
      if (col < p.cols) {
        const size_t off = (size_t)row * p.cols + col;
        float4 part[kPeerMaxTp];
#pragma unroll
        for (int r = 0; r < kPeerMaxTp; ++r)
          if (r < p.tp) part[r] = (r == p.rank) ? *reinterpret_cast<const float4*>(p.data[r] + off) : ld_peer_f4(p.data[r] + off);
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < kPeerMaxTp; ++r)   // rank order on every rank: all ranks get the same bits
          if (r < p.tp) { sum.x += part[r].x; sum.y += part[r].y; sum.z += part[r].z; sum.w += part[r].w; }
        float4 v = *reinterpret_cast<float4*>(p.x + off);
        v.x += sum.x; v.y += sum.y; v.z += sum.z; v.w += sum.w;
        *reinterpret_cast<float4*>(p.x + off) = v;
        if (p.emit_base) {
          float y[4] = {v.x, v.y, v.z, v.w};
          if (p.emit_norm) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(p.emit_norm + col));
            y[0] *= w.x; y[1] *= w.y; y[2] *= w.z; y[3] *= w.w;
          }
          unsigned short a[4], b[4], c[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) pi_split3(y[j], a[j], b[j], c[j]);
          unsigned short* q = p.emit_base + off;
          *reinterpret_cast<uint2*>(q) = make_uint2((uint32_t)a[0] | ((uint32_t)a[1] << 16), (uint32_t)a[2] | ((uint32_t)a[3] << 16));
          *reinterpret_cast<uint2*>(q + p.emit_plane_stride) = make_uint2((uint32_t)b[0] | ((uint32_t)b[1] << 16), (uint32_t)b[2] | ((uint32_t)b[3] << 16));
          *reinterpret_cast<uint2*>(q + 2 * p.emit_plane_stride) = make_uint2((uint32_t)c[0] | ((uint32_t)c[1] << 16), (uint32_t)c[2] | ((uint32_t)c[3] << 16));
          sq = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
        }
      }
      if (p.emit_sumsq) {   // sum of squares of this chunk of the row, fixed order
        sq = pi_warp_sum(sq);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = sq;
        __syncthreads();
        if (threadIdx.x == 0) {
          float t = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) t += s_red[i];
          p.emit_sumsq[(size_t)seg * p.emit_sumsq_stride + row] = t;
        }
        __syncthreads();
      }
    }
  }
  // the last CTA to finish advances the epoch of this slot for the next exchange on it
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int t = atomicAdd(p.ticket, 1u);
    if (t == gridDim.x - 1) {
      *p.ticket = 0u;
      *reinterpret_cast<volatile unsigned long long*>(p.epoch) = e;
    }
  }
}

size_t peer_flags_offset(size_t slot_floats, int tp) { return (size_t)kPeerSlots * tp * slot_floats * sizeof(float); }
}  // namespace

extern "C" pi_status pi_tp_peer_export(pi_ctx* ctx, size_t max_floats, void* handle_out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, handle_out && max_floats > 0, "null pointer or empty buffer");
  PI_REQUIRE(ctx, ctx->tp > 1 && ctx->tp <= kPeerMaxTp, "the peer path needs a tensor-parallel context");
  PI_REQUIRE(ctx, !ctx->peer.base, "the peer buffers of this context exist already");
  static_assert(sizeof(cudaIpcMemHandle_t) == PI_TP_PEER_HANDLE_BYTES, "cudaIpcMemHandle_t is 64 bytes");
  const size_t slot_floats = (max_floats + 63) / 64 * 64;
  const size_t bytes = peer_flags_offset(slot_floats, ctx->tp) + (kPeerSlots * kPeerMaxTp + kPeerSlots) * sizeof(unsigned long long) +
                       kPeerSlots * sizeof(unsigned int) + 64;
  PI_CUDA(ctx, cudaMalloc(&ctx->peer.base, bytes));
  PI_CUDA(ctx, cudaMemset(ctx->peer.base, 0, bytes));
  ctx->peer.slot_floats = slot_floats;
  cudaIpcMemHandle_t h;
  PI_CUDA(ctx, cudaIpcGetMemHandle(&h, ctx->peer.base));
  memcpy(handle_out, &h, sizeof(h));
  return PI_OK;
}

extern "C" pi_status pi_tp_peer_import(pi_ctx* ctx, const void* handles) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, handles && ctx->peer.base, "call pi_tp_peer_export first");
  const unsigned char* all = static_cast<const unsigned char*>(handles);
  for (int r = 0; r < ctx->tp; ++r) {
    void* base = ctx->peer.base;
    if (r != ctx->rank) {
      cudaIpcMemHandle_t h;
      memcpy(&h, all + (size_t)r * sizeof(h), sizeof(h));
      PI_CUDA(ctx, cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
      ctx->peer.mapped[r] = base;
    }
    ctx->peer.data[r] = static_cast<float*>(base);
    ctx->peer.flags[r] = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(base) + peer_flags_offset(ctx->peer.slot_floats, ctx->tp));
  }
  ctx->peer.next_slot = 0;
  ctx->peer.ready = true;
  return PI_OK;
}

extern "C" void* pi_tp_peer_base(const pi_ctx* ctx) { return ctx ? ctx->peer.base : nullptr; }

extern "C" pi_status pi_tp_peer_import_pointers(pi_ctx* ctx, void* const* bases) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, bases && ctx->peer.base, "call pi_tp_peer_export first");
  PI_REQUIRE(ctx, bases[ctx->rank] == ctx->peer.base, "entry %d of the pointer table must be this context's own buffer", ctx->rank);
  for (int r = 0; r < ctx->tp; ++r) {
    PI_REQUIRE(ctx, bases[r] != nullptr, "rank %d has no buffer", r);
    ctx->peer.data[r] = static_cast<float*>(bases[r]);
    ctx->peer.flags[r] = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(bases[r]) + peer_flags_offset(ctx->peer.slot_floats, ctx->tp));
  }
  ctx->peer.next_slot = 0;
  ctx->peer.ready = true;
  return PI_OK;
}

extern "C" pi_status pi_tp_exchange_add(pi_ctx* ctx, const float* partial_dev, float* x_dev, int rows, int cols) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, partial_dev && x_dev && rows > 0 && cols > 0, "null pointer or empty matrix");
  const size_t n = (size_t)rows * cols;
  if (ctx->tp == 1) return pi_launch_add(ctx, x_dev, partial_dev, n);
  if (pi_tp_peer_usable(ctx, n) && cols % 4 == 0 && (uintptr_t)x_dev % 16 == 0) {
    PI_CUDA(ctx, cudaMemcpyAsync(pi_tp_peer_slot(ctx), partial_dev, n * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    return pi_tp_peer_reduce_add(ctx, x_dev, rows, cols);
  }
  PI_TRY(pi_reserve(ctx, &ctx->staging_in, n * sizeof(float)));
  float* tmp = static_cast<float*>(ctx->staging_in.ptr);
  PI_CUDA(ctx, cudaMemcpyAsync(tmp, partial_dev, n * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
  PI_TRY(pi_tp_all_reduce_sum(ctx, tmp, n));
  return pi_launch_add(ctx, x_dev, tmp, n);
}

bool pi_tp_peer_usable(const pi_ctx* ctx, size_t n) {
  return ctx->tp > 1 && ctx->peer.ready && n <= ctx->peer.slot_floats && n % 4 == 0;
}

// Region `region` of the slot of the next exchange in rank `owner`'s buffer.
static float* peer_region(const pi_ctx* ctx, int owner, int slot, int region) {
  return ctx->peer.data[owner] + ((size_t)slot * ctx->tp + region) * ctx->peer.slot_floats;
}

float* pi_tp_peer_slot(pi_ctx* ctx) { return peer_region(ctx, ctx->rank, ctx->peer.next_slot, ctx->rank); }

int pi_tp_peer_push_targets(pi_ctx* ctx, float** out) {
  int n = 0;
  for (int r = 0; r < ctx->tp; ++r)
    if (r != ctx->rank) out[n++] = peer_region(ctx, r, ctx->peer.next_slot, ctx->rank);
  ctx->peer.pushed = true;   // the next exchange finds every rank's partial sums in its own memory
  return n;
}

pi_status pi_tp_peer_reduce_add(pi_ctx* ctx, float* x, int rows, int cols, pi_act_planes* emit, const float* emit_norm_weight,
                                float emit_norm_eps) {
  const size_t n = (size_t)rows * cols;
  PI_REQUIRE(ctx, pi_tp_peer_usable(ctx, n) && cols % 4 == 0 && (uintptr_t)x % 16 == 0, "the peer exchange is not set up for %zu values", n);
  pi_prof_scope prof(ctx, PI_PROF_COLLECTIVE);
  const int slot = ctx->peer.next_slot;
  ctx->peer.next_slot ^= 1;
  PeerReduceParams p = {};
  p.x = x;
  p.rows = rows;
  p.cols = cols;
  p.tp = ctx->tp;
  p.rank = ctx->rank;
  p.slot = slot;
  const bool pushed = ctx->peer.pushed;
  ctx->peer.pushed = false;
  for (int r = 0; r < ctx->tp; ++r) {
    p.data[r] = peer_region(ctx, pushed ? ctx->rank : r, slot, r);
    p.flags[r] = ctx->peer.flags[r];
  }
  unsigned long long* epoch = ctx->peer.flags[ctx->rank] + kPeerSlots * kPeerMaxTp;
  p.epoch = epoch + slot;
  p.ticket = reinterpret_cast<unsigned int*>(epoch + kPeerSlots) + slot;
  p.err_flag = ctx->dev_err;
  p.spin_limit = ctx->peer_spin_limit ? ctx->peer_spin_limit : (1u << 22);
  const int cpr = (cols + kPeerChunk - 1) / kPeerChunk;
  if (emit) {
    PI_REQUIRE(ctx, emit->base && emit->K == cols && emit->plane_stride % 4 == 0 && (uintptr_t)emit->base % 8 == 0,
               "planes of %d columns are needed", cols);
    p.emit_base = reinterpret_cast<unsigned short*>(emit->base);
    p.emit_plane_stride = emit->plane_stride;
    p.emit_norm = emit_norm_weight;
    emit->row_scale = nullptr;
    emit->sumsq_tiles = 0;
    if (emit_norm_weight) {
      PI_REQUIRE(ctx, emit->sumsq && emit->sumsq_stride >= (size_t)rows && (uintptr_t)emit_norm_weight % 16 == 0,
                 "emit with a norm weight needs a sums-of-squares buffer");
      p.emit_sumsq = emit->sumsq;
      p.emit_sumsq_stride = emit->sumsq_stride;
      emit->sumsq_tiles = cpr;
      emit->eps = emit_norm_eps;
    }
  }
  const unsigned grid = (unsigned)std::min<size_t>((size_t)rows * cpr, (size_t)ctx->sm_count);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(std::max(grid, 1u));
  cfg.blockDim = dim3(256);
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, tp_peer_reduce_add_kernel, p);
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "peer exchange launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  return PI_OK;
}
