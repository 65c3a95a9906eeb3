// Internal declarations shared by the translation units of libpaged_infer_cuda.so.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <vector>

#include "../../include/paged_infer_cuda.h"

#define PI_WARP 32

// ---- error plumbing -----------------------------------------------------------
pi_status pi_fail(pi_ctx* ctx, pi_status code, const char* fmt, ...);
void pi_set_global_error(const char* msg);

#define PI_CUDA(ctx, expr)                                                                        \
  do {                                                                                            \
    cudaError_t _e = (expr);                                                                      \
    if (_e != cudaSuccess)                                                                        \
      return pi_fail((ctx), _e == cudaErrorMemoryAllocation ? PI_ERR_OOM : PI_ERR_CUDA,           \
                     "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
  } while (0)

#define PI_CHECK_LAUNCH(ctx)                                                                           \
  do {                                                                                                 \
    cudaError_t _e = cudaGetLastError();                                                               \
    if (_e != cudaSuccess)                                                                             \
      return pi_fail((ctx), PI_ERR_CUDA, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e),   \
                     __FILE__, __LINE__);                                                              \
    (ctx)->launches++;                                                                                 \
  } while (0)

#define PI_REQUIRE(ctx, cond, ...)                                     \
  do {                                                                 \
    if (!(cond)) return pi_fail((ctx), PI_ERR_INVALID_ARG, __VA_ARGS__); \
  } while (0)

// First line of an API entry point: a null context is an argument error; a host thread whose current device is not
// the context's is switched to it (every launch, copy and allocation below goes to the current device).
#define PI_ENTER(ctx)                              \
  do {                                             \
    if (!(ctx)) return PI_ERR_INVALID_ARG;         \
    pi_status _se = pi_enter(ctx);                 \
    if (_se != PI_OK) return _se;                  \
  } while (0)

#define PI_TRY(expr)               \
  do {                             \
    pi_status _s = (expr);         \
    if (_s != PI_OK) return _s;    \
  } while (0)

constexpr int PI_DEV_ERR_WORDS = 16;

// ---- context ------------------------------------------------------------------
// A growable device buffer owned by the context (scratch that outlives a call).
struct pi_buffer {
  void* ptr = nullptr;
  size_t bytes = 0;
};

struct pi_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int sm_count = 148;
  size_t smem_optin = 0;
  std::string err;
  uint64_t launches = 0;
  int* dev_err = nullptr;   // device words: [0] set by a kernel that gave up (bounded wait ran out, inconsistent input), [1..] its record

  // tensor parallelism
  int rank = 0, tp = 1;
  void* nccl_comm = nullptr;  // ncclComm_t
  // Peer-memory exchange for the row-split projections (optional, set up with pi_tp_peer_export/import): every rank
  // owns `slots` buffers of partial sums that its peers read directly over NVLink, plus arrival flags they write.
  struct {
    bool ready = false;
    size_t slot_floats = 0;
    void* base = nullptr;                       // one allocation: [2 slots of floats | flags[2][8] | epoch[2] | ticket[2]]
    float* data[8] = {};                        // slot 0 of every rank's buffer (own rank: local pointer)
    unsigned long long* flags[8] = {};          // every rank's flag array
    void* mapped[8] = {};                       // what cudaIpcOpenMemHandle returned (to close)
    int next_slot = 0;
    bool pushed = false;                        // the partial sums of the next exchange were pushed into every rank's buffer
  } peer;
  uint32_t peer_spin_limit = 0;   // polls a rank waits for a peer's partial sums; 0 = the default (about a second)

  // options
  bool opt_tensor_gemm = true;
  bool opt_graph = true;
  bool opt_pdl = true;
  int opt_gemv_max_m = 4;
  int opt_attn_shared = 1;   // entries that share one block table: 0 decode kernel, 1 shared-table kernel when it fills the GPU, 2 always, 3 always and on the mma.sync kernel
  int opt_attn_tma = 1;   // 0 direct loads, 1 tile-at-a-time kernel (block size 16) over a TMA ring, 2 per-token kernel over a TMA ring
  // batched decode with many tiles over one flat tile list (an equal range per resident warp): 0 never, 1 inside a
  // model forward, where one work list serves all layers of the step, 2 also for a single pi_paged_attention call
  // (which then pays for its own work-list kernel: slower than the per-entry grid, there for tests)
  int opt_attn_flat = 1;
  bool opt_tp_push = true;  // tensor parallel, peer path: row-split projections push their partial sums into every rank's buffer
  int opt_fuse_planes = 1;  // model forward: projections hand their result to the next one as bf16 planes (no split kernel)

  // per-kernel-class timing with CUDA events on this stream (off by default)
  bool prof_on = false;
  std::vector<cudaEvent_t> prof_events;  // 2 per recorded launch
  std::vector<int> prof_class;
  size_t prof_used = 0;

  // scratch
  pi_buffer staging_in, staging_out;   // device copies of host arguments / results
  pi_buffer attn_tables;               // block tables + per-entry (len, pos, start)
  pi_buffer attn_partial;              // split-KV partial (m, l, acc)
  pi_buffer attn_plan;                 // flat work list of the step: segment ranges, segments, merge info, counters
  pi_buffer gemm_act;                  // bf16 activation planes (+ row factors) for the tensor GEMM
  std::vector<uint8_t> scratch_block_marks;   // host: physical blocks written by the step being staged
  void* pinned = nullptr;              // pinned host staging
  size_t pinned_bytes = 0;
};

// Brackets one launch (or one short launch sequence) with events while profiling is on.
struct pi_prof_scope {
  pi_ctx* ctx;
  long slot;
  pi_prof_scope(pi_ctx* c, int cls);
  ~pi_prof_scope();
};

pi_status pi_enter(pi_ctx* ctx);
pi_status pi_reserve(pi_ctx* ctx, pi_buffer* buf, size_t bytes);
pi_status pi_reserve_pinned(pi_ctx* ctx, size_t bytes);

// ---- projections ----------------------------------------------------------------
struct pi_linear {
  int kind = PI_INT8;          // PI_F32 / PI_INT8 / PI_BF16
  pi_split split = PI_SPLIT_NONE;
  size_t full_rows = 0, full_cols = 0;
  size_t rows = 0, cols = 0;   // local shard
  size_t ld = 0;               // row stride in elements (rows start 16-byte aligned, zero padded)
  void* w = nullptr;           // [rows][ld]
  float* scales = nullptr;     // [rows] (int8 only)
  bool owns = true;
};

enum pi_epilogue {
  PI_EPI_STORE = 0,     // out[m][r] = v
  PI_EPI_ADD = 1,       // out[m][r] += v           (residual add)
  PI_EPI_SWIGLU = 2     // rows interleaved gate/up: out[m][r/2] = silu(v[2i]) * v[2i+1]
};

// An activation matrix in the form the tensor-core GEMM consumes: three bf16 planes whose sum is the f32 value
// exactly (plane 0 = bf16(y), plane 1 = bf16(y - p0), plane 2 = bf16(y - p0 - p1)), plus a per-row factor that the
// consumer's epilogue multiplies back in.  For an RMS-normalised input y = x * norm_weight is what the planes hold and
// the factor is 1/rms(x): either given directly (`row_scale`) or as per-tile partial sums of x^2 (`sumsq`), in which
// case the factor is 1/sqrt(sum_over_tiles / K + eps).  Both null: factor 1.
struct pi_act_planes {
  __nv_bfloat16* base = nullptr;   // [3][rows_cap][K]
  size_t plane_stride = 0;         // elements between planes
  int K = 0;
  float* row_scale = nullptr;      // [rows]
  float* sumsq = nullptr;          // [sumsq_tiles][sumsq_stride]
  int sumsq_tiles = 0;
  size_t sumsq_stride = 0;
  float eps = 0.f;
};

struct pi_kv_pool;
struct pi_attn_batch;
// Rotary embedding + KV write folded into the epilogue of the fused [q;k;v] projection (tensor-core path): the
// kernel rotates the q and k heads (math::rope_rotate, src/math.rs:344-367), leaves q in `out` for the attention and
// scatters k and v of every row into the pool at that row's position (write skipped when the logical block is not
// mapped, src/model.rs:1094).  Ask pi_gemm_tc_can_rope first.
struct pi_rope_kv {
  int num_heads = 0, num_kv_heads = 0, head_dim = 0, style = 0;
  const float* rope_cos = nullptr;   // [positions][head_dim/2]
  const float* rope_sin = nullptr;
  pi_kv_pool* pool = nullptr;
  int layer = 0;
  const pi_attn_batch* batch = nullptr;
};

struct pi_linear_args {
  const float* x = nullptr;   // [M][x_stride]
  size_t x_stride = 0;
  float* out = nullptr;       // [M][out_stride]
  size_t out_stride = 0;
  int M = 1;
  pi_epilogue epi = PI_EPI_STORE;
  const float* norm_weight = nullptr;  // fused RMSNorm prologue when non-null
  float norm_eps = 0.f;
  // Tensor-core path only.  `in_planes`: x (after norm_weight, if any) is already available as planes, skip the
  // split.  `emit`: besides `out`, write the result as planes for the next projection (base, plane_stride, K and the
  // sumsq buffer are the caller's; with `emit_norm_weight` the planes hold out * weight and the kernel fills the
  // per-tile sums of out^2 and sets sumsq_tiles).  Ask pi_gemm_tc_can_emit first.
  const pi_act_planes* in_planes = nullptr;
  pi_act_planes* emit = nullptr;
  const float* emit_norm_weight = nullptr;
  float emit_norm_eps = 0.f;
  const pi_rope_kv* rope = nullptr;
  // Tensor-core path, plain store epilogue only: the result is also stored at the same offsets under these bases
  // (peer memory of the other tensor-parallel ranks).
  float* out_also[8] = {};
  int n_out_also = 0;
};

// CUDA-core dequant GEMV/GEMM (any shape, any M).
pi_status pi_launch_gemv(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a);
// tcgen05 tensor-core GEMM for int8 weights (returns PI_ERR_UNSUPPORTED when the shape does not fit).
pi_status pi_launch_gemm_tc(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a);
bool pi_gemm_tc_supported(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a);
// True when pi_linear_forward would take the tensor-core path for this call.
bool pi_gemm_tc_will_run(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a);
// True when that launch can also emit planes (and, with a norm weight, the partial sums of squares).
bool pi_gemm_tc_can_emit(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, bool with_norm);
// True when that launch can also apply the rotary embedding and write K/V into the pool.
bool pi_gemm_tc_can_rope(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, const pi_rope_kv& r);
// The same for the CUDA-core path (any head_dim that is even).
bool pi_gemv_can_rope(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, const pi_rope_kv& r);
// The activation split on its own (what the GEMM runs first when it is not given planes): x -> planes in `dst`.
pi_status pi_launch_act_split(pi_ctx* ctx, const float* x, size_t x_stride, const float* norm_weight, float eps, int M, int K,
                              pi_act_planes* dst);
// Dispatch between the two.
pi_status pi_linear_forward(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a);

pi_status pi_linear_alloc(pi_ctx* ctx, int kind, size_t full_rows, size_t full_cols, pi_split split, pi_linear** out);
// Copy a [rows x cols] host or device matrix (row stride src_ld elements) into the padded device layout.
pi_status pi_linear_fill(pi_ctx* ctx, pi_linear* lin, const void* src, size_t src_ld, bool src_on_device);
pi_status pi_launch_quantize(pi_ctx* ctx, const float* w_dev, size_t w_ld, size_t rows, size_t cols, int8_t* q_dev,
                             size_t q_ld, float* scales_dev);

// ---- KV pool ----------------------------------------------------------------------
// Device layout: [layer][block][kv_head][k|v][token][head_dim] f32, so one
// (block, kv_head) K tile is block_size*head_dim contiguous floats with its V
// tile right behind it, and one block of one layer is still one contiguous span.
struct pi_kv_pool {
  pi_kv_layout L;
  float* data = nullptr;
  size_t floats = 0;
  __host__ __device__ size_t block_stride() const { return (size_t)L.block_size * L.num_kv_heads * 2 * L.head_dim; }
};

__host__ __device__ inline size_t pi_kv_tile_offset(const pi_kv_layout& L, int layer, int block, int kv_head, int is_v) {
  return ((((size_t)layer * L.num_blocks + block) * L.num_kv_heads + kv_head) * 2 + is_v) * ((size_t)L.block_size * L.head_dim);
}

// ---- attention ----------------------------------------------------------------------
struct pi_attn_batch {
  const int32_t* tables = nullptr;  // device [B][max_blocks]
  int max_blocks = 0;
  const int32_t* lens = nullptr;    // device [B]
  const int32_t* pos = nullptr;     // device [B]
  const int32_t* start = nullptr;   // device [B]
  // device [B]: logical blocks below this index are complete and will not be written by anything queued after the
  // upload (the position the host passed, in blocks; 0 for an entry with a window start): a kernel may fetch them
  // before it has waited for the kernel ahead of it.  Never updated on the device.
  const int32_t* safe_lb = nullptr;
  int B = 0;
  int max_window_blocks = 0;        // host-side bound on blocks any window touches
  long total_window_blocks = 0;     // host-side sum
  bool shared_table = false;        // every entry maps the same table row (a prefill chunk, a speculative verify group)
  int shared_len = 0;               // ... of this many blocks
  // Flat work list of the step (pi_attention_prepare): warp slots it was cut for (0: none, use the per-entry grid),
  // partial slots, and the device arrays the planning kernel fills.  Set per step, hence mutable.
  mutable int flat_warps = 0;
  mutable size_t flat_slots = 0;
  mutable void* flat_hdr = nullptr;
  mutable bool flat_settled = false;   // every kernel queued since the planning kernel has waited for its predecessor
  mutable void* flat_segs = nullptr;
  mutable void* flat_comb = nullptr;
  mutable int* flat_counters = nullptr;
};
pi_status pi_upload_attn_batch(pi_ctx* ctx, const int32_t* tables_host, int max_blocks, const int32_t* lens_host,
                               const int32_t* pos_host, const int32_t* start_host, int B, int block_size, int num_blocks,
                               pi_attn_batch* out);
// `emit` (optional): when the KV axis is split and a merge kernel runs anyway, that kernel also writes the output as
// bf16 planes (row factor 1) for the projection that follows; *emitted tells whether it did.
bool pi_attention_shared_usable(const pi_ctx* ctx, const pi_kv_pool* pool, int num_heads, const float* q, size_t q_stride,
                                const float* out, size_t out_stride, const pi_attn_batch& batch);
bool pi_attention_shared_tc_usable(const pi_ctx* ctx, const pi_kv_pool* pool, int num_heads, const float* q, size_t q_stride,
                                   const float* out, size_t out_stride);
pi_status pi_launch_attention_shared_tc(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q,
                                        size_t q_stride, float* out, size_t out_stride, const pi_attn_batch& batch);
pi_status pi_launch_attention_shared(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q,
                                     size_t q_stride, float* out, size_t out_stride, const pi_attn_batch& batch);
pi_status pi_attention_prepare(pi_ctx* ctx, const pi_kv_pool* pool, int num_heads, const pi_attn_batch& batch);
pi_status pi_launch_attention_flat(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q,
                                   size_t q_stride, float* out, size_t out_stride, const pi_attn_batch& batch,
                                   pi_act_planes* emit, bool* emitted);
pi_status pi_launch_attention(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q,
                              size_t q_stride, float* out, size_t out_stride, const pi_attn_batch& batch,
                              pi_act_planes* emit = nullptr, bool* emitted = nullptr);

// ---- glue ----------------------------------------------------------------------------
pi_status pi_launch_embed(pi_ctx* ctx, const uint16_t* table_bf16, int vocab, int hidden, const uint32_t* tokens_dev,
                          int B, float* x);
pi_status pi_launch_rms_norm(pi_ctx* ctx, float* x, size_t stride, const float* weight, int rows, int n, float eps);
// Rotate q (in place) and k, then scatter k and v into the pool. qkv is [B][qkv_stride] = [q | k | v].
pi_status pi_launch_rope_kv_write(pi_ctx* ctx, float* qkv, size_t qkv_stride, int num_heads, int num_kv_heads,
                                  int head_dim, const float* rope_cos, const float* rope_sin, int style,
                                  pi_kv_pool* pool, int layer, const pi_attn_batch& batch);
pi_status pi_launch_rope(pi_ctx* ctx, float* x, size_t stride, int heads, int head_dim, const int32_t* pos_dev,
                         const float* rope_cos, const float* rope_sin, int style, int rows);
pi_status pi_launch_swiglu(pi_ctx* ctx, float* gate, const float* up, size_t n);
pi_status pi_launch_add(pi_ctx* ctx, float* x, const float* y, size_t n);
pi_status pi_launch_argmax(pi_ctx* ctx, const float* logits, size_t stride, int rows, int n, uint32_t* out);
pi_status pi_launch_copy_block(pi_ctx* ctx, pi_kv_pool* pool, int src, int dst);
pi_status pi_launch_kv_relayout(pi_ctx* ctx, const pi_kv_pool* pool, float* ref_layout, bool to_reference);
// N(0, std) from a counter-based generator keyed by (seed, stream id); element 2i and 2i+1 come from
// counter pair_offset + i, so any even-aligned slice of a tensor reproduces the whole tensor's values.
pi_status pi_launch_fill_normal(pi_ctx* ctx, float* out, size_t n, uint64_t seed, uint64_t stream_id,
                                uint64_t pair_offset, float std);
pi_status pi_launch_f32_to_bf16(pi_ctx* ctx, const float* in, uint16_t* out, size_t n);
pi_status pi_launch_bf16_to_f32(pi_ctx* ctx, const uint16_t* in, size_t in_ld, float* out, size_t out_ld, size_t rows, size_t cols);

// Host rotary table exactly as the reference builds it (f32 powf/sinf/cosf of the host libm).
void pi_host_rope_table(int pos, int head_dim, float theta, float* cos_out, float* sin_out);

// ---- tensor parallel -------------------------------------------------------------------
pi_status pi_tp_init(pi_ctx* ctx, const void* unique_id);
void pi_tp_destroy(pi_ctx* ctx);
pi_status pi_tp_all_reduce_sum(pi_ctx* ctx, float* buf, size_t n);
pi_status pi_tp_all_gather(pi_ctx* ctx, const void* send, void* recv, size_t bytes_per_rank);
// Peer path: where this rank's next row-split projection must write its [n] partial sums, and the kernel that waits
// for all ranks' partials of that slot, adds them in rank order and adds the sum to x.
bool pi_tp_peer_usable(const pi_ctx* ctx, size_t n);
float* pi_tp_peer_slot(pi_ctx* ctx);
// Push variant: where the same partial sums go in the other ranks' buffers (tp - 1 pointers into peer memory, written
// to `out`; returns their number).  The projection stores its result there as well as in pi_tp_peer_slot(); the next
// pi_tp_peer_reduce_add then reads every rank's partial sums from local memory.
int pi_tp_peer_push_targets(pi_ctx* ctx, float** out);
// `emit` (optional): also write the new rows of x as planes (times emit_norm_weight, with the per-chunk sums of
// squares the consumer turns into 1/rms), so that the projection that follows needs no split kernel.
pi_status pi_tp_peer_reduce_add(pi_ctx* ctx, float* x, int rows, int cols, pi_act_planes* emit = nullptr,
                                const float* emit_norm_weight = nullptr, float emit_norm_eps = 0.f);

// ---- device helpers ----------------------------------------------------------------------
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is per device and slow: what each launcher has already been granted,
// per device of the calling context.
struct pi_smem_grant {
  size_t bytes[64] = {};
  size_t& of(const pi_ctx* ctx) { return bytes[(unsigned)ctx->device & 63u]; }
};

#ifdef __CUDACC__
// y = p0 + p1 + p2 exactly, each a bf16 (each remainder has at most 16, then 8 significant bits left).
__device__ __forceinline__ void pi_split3(float y, unsigned short& p0, unsigned short& p1, unsigned short& p2) {
  const __nv_bfloat16 a = __float2bfloat16_rn(y);
  const float r1 = y - __bfloat162float(a);
  const __nv_bfloat16 b = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(b);
  const __nv_bfloat16 c = __float2bfloat16_rn(r2);
  p0 = __bfloat16_as_ushort(a);
  p1 = __bfloat16_as_ushort(b);
  p2 = __bfloat16_as_ushort(c);
}

__device__ __forceinline__ float pi_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float pi_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float pi_bf16_bits_to_f32(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
// Programmatic dependent launch: wait for the producer grid's memory, and allow
// the consumer grid to start its prologue.
// Every kernel of this library guards its first dependent access with this call, so the next kernel in
// the stream may be released right here: it can then run its own independent prologue (barrier set-up, TMEM
// allocation, weight prefetch) while this grid is still working, and blocks in its own wait until this grid has
// completed.  The dependent grid is only released once every CTA of this grid has passed this point or exited.
__device__ __forceinline__ void pi_grid_dependency_wait() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pi_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// The other order: nothing queued behind this grid starts before the grid ahead of it has completed.  One such kernel
// in a chain is a fence for early reads: whatever ran before it is complete in the eyes of EVERY later kernel, even in
// the part of a later kernel that precedes its own dependency wait.
__device__ __forceinline__ void pi_grid_dependency_wait_strict() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif
