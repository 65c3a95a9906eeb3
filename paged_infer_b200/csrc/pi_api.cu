// C-ABI entry points: context, quantiser, projections, KV pool, attention and
// the host-buffer glue calls.  The model forward lives in pi_model.cu.
#include <stdarg.h>
#include <string.h>

#include <algorithm>
#include <new>

#include "pi_common.cuh"

namespace {
thread_local std::string g_create_error;
}

void pi_set_global_error(const char* msg) { g_create_error = msg ? msg : ""; }

pi_status pi_fail(pi_ctx* ctx, pi_status code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  else g_create_error = buf;
  return code;
}

pi_prof_scope::pi_prof_scope(pi_ctx* c, int cls) : ctx(c), slot(-1) {
  if (!c->prof_on || c->prof_used >= (1u << 16)) return;
  if (c->prof_events.size() < 2 * (c->prof_used + 1)) {
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    c->prof_events.push_back(a);
    c->prof_events.push_back(b);
  }
  slot = (long)c->prof_used++;
  c->prof_class.push_back(cls);
  cudaEventRecord(c->prof_events[2 * slot], c->stream);
}
pi_prof_scope::~pi_prof_scope() {
  if (slot >= 0) cudaEventRecord(ctx->prof_events[2 * slot + 1], ctx->stream);
}

pi_status pi_enter(pi_ctx* ctx) {
  int dev = -1;
  if (cudaGetDevice(&dev) == cudaSuccess && dev == ctx->device) return PI_OK;
  PI_CUDA(ctx, cudaSetDevice(ctx->device));
  return PI_OK;
}

pi_status pi_reserve(pi_ctx* ctx, pi_buffer* buf, size_t bytes) {
  if (bytes <= buf->bytes) return PI_OK;
  // The old allocation may still be in use by queued kernels.
  if (buf->ptr) {
    PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    PI_CUDA(ctx, cudaFree(buf->ptr));
    buf->ptr = nullptr;
    buf->bytes = 0;
  }
  const size_t want = std::max(bytes, (size_t)4096);
  PI_CUDA(ctx, cudaMalloc(&buf->ptr, want));
  buf->bytes = want;
  return PI_OK;
}

pi_status pi_reserve_pinned(pi_ctx* ctx, size_t bytes) {
  // Pinned staging is reused by every call: wait for the previous user's copies.
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (bytes <= ctx->pinned_bytes) return PI_OK;
  if (ctx->pinned) PI_CUDA(ctx, cudaFreeHost(ctx->pinned));
  ctx->pinned = nullptr;
  ctx->pinned_bytes = 0;
  const size_t want = std::max(bytes, (size_t)1 << 16);
  PI_CUDA(ctx, cudaMallocHost(&ctx->pinned, want));
  ctx->pinned_bytes = want;
  return PI_OK;
}

static pi_status check_device_flag(pi_ctx* ctx) {
  // word 0: the code of the kernel that gave up; words 1..: that kernel's own record of what it saw (first reporter only)
  int rec[PI_DEV_ERR_WORDS] = {};
  PI_CUDA(ctx, cudaMemcpyAsync(rec, ctx->dev_err, sizeof(rec), cudaMemcpyDeviceToHost, ctx->stream));
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  const int flag = rec[0];
  if (flag != 0) {
    PI_CUDA(ctx, cudaMemsetAsync(ctx->dev_err, 0, sizeof(rec), ctx->stream));
    if (flag >= 11 && flag <= 13)
      return pi_fail(ctx, PI_ERR_CUDA, "the attention work list of the step is inconsistent (code %d: warp slot %d, segments %d..%d, "
                                      "entry %d, kv head %d, blocks %d..%d, physical block %d, item %d); nothing was read through it",
                     flag, rec[2], rec[3], rec[4], rec[5], rec[6], rec[7], rec[8], rec[9], rec[10]);
    if (flag == 9) {
      // a peer never delivered its partial sums: the slots of the ranks are out of step from here on, so the
      // peer-memory exchange is retired and later steps go through NCCL (or fail loudly without a communicator)
      ctx->peer.ready = false;
      return pi_fail(ctx, PI_ERR_TIMEOUT, "a tensor-parallel peer did not deliver its partial sums in time (code 9); "
                                          "the results of this step are invalid and the peer-memory exchange is disabled");
    }
    return pi_fail(ctx, PI_ERR_TIMEOUT, "a kernel's bounded wait ran out (code %d)", flag);
  }
  return PI_OK;
}

extern "C" {

const char* pi_version(void) { return "paged_infer_cuda 0.1 (sm_100a)"; }

const char* pi_last_error(const pi_ctx* ctx) { return ctx ? ctx->err.c_str() : g_create_error.c_str(); }

static pi_status ctx_create_common(int device, void* stream, pi_ctx** out) {
  if (!out) return pi_fail(nullptr, PI_ERR_INVALID_ARG, "out is NULL");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return pi_fail(nullptr, PI_ERR_CUDA, "no CUDA device available: %s (this library has no CPU fallback)",
                   cudaGetErrorString(e));
  if (device < 0 || device >= count) return pi_fail(nullptr, PI_ERR_INVALID_ARG, "device %d of %d", device, count);
  e = cudaSetDevice(device);
  if (e != cudaSuccess) return pi_fail(nullptr, PI_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return pi_fail(nullptr, PI_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return pi_fail(nullptr, PI_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                   prop.major, prop.minor);
  pi_ctx* ctx = new (std::nothrow) pi_ctx();
  if (!ctx) return pi_fail(nullptr, PI_ERR_OOM, "host allocation failed");
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->smem_optin = prop.sharedMemPerBlockOptin;
  if (stream) {
    ctx->stream = static_cast<cudaStream_t>(stream);
  } else {
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
      delete ctx;
      return pi_fail(nullptr, PI_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e));
    }
    ctx->own_stream = true;
  }
  e = cudaMalloc(&ctx->dev_err, PI_DEV_ERR_WORDS * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(ctx->dev_err, 0, PI_DEV_ERR_WORDS * sizeof(int));
  if (e != cudaSuccess) {
    delete ctx;
    return pi_fail(nullptr, PI_ERR_CUDA, "context allocation: %s", cudaGetErrorString(e));
  }
  *out = ctx;
  return PI_OK;
}

pi_status pi_ctx_create(int device, void* stream, pi_ctx** out) { return ctx_create_common(device, stream, out); }

pi_status pi_ctx_create_tp(int device, void* stream, int rank, int tp, const void* nccl_unique_id, pi_ctx** out) {
  if (!(tp == 1 || tp == 2 || tp == 4 || tp == 8) || rank < 0 || rank >= tp)
    return pi_fail(nullptr, PI_ERR_INVALID_ARG, "tensor-parallel rank %d of %d (tp must be 1, 2, 4 or 8)", rank, tp);
  PI_TRY(ctx_create_common(device, stream, out));
  (*out)->rank = rank;
  (*out)->tp = tp;
  if (tp > 1 && nccl_unique_id) {
    pi_status s = pi_tp_init(*out, nccl_unique_id);
    if (s != PI_OK) {
      g_create_error = (*out)->err;
      pi_ctx_destroy(*out);
      *out = nullptr;
      return s;
    }
  }
  return PI_OK;
}

void pi_ctx_destroy(pi_ctx* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  pi_tp_destroy(ctx);
  for (pi_buffer* b : {&ctx->staging_in, &ctx->staging_out, &ctx->attn_tables, &ctx->attn_partial, &ctx->attn_plan, &ctx->gemm_act})
    if (b->ptr) cudaFree(b->ptr);
  if (ctx->pinned) cudaFreeHost(ctx->pinned);
  for (cudaEvent_t e : ctx->prof_events) cudaEventDestroy(e);
  if (ctx->dev_err) cudaFree(ctx->dev_err);
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
}

pi_status pi_ctx_synchronize(pi_ctx* ctx) {
  PI_ENTER(ctx);
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return check_device_flag(ctx);
}

uint64_t pi_ctx_kernel_launches(const pi_ctx* ctx) { return ctx ? ctx->launches : 0; }
void pi_ctx_reset_kernel_launches(pi_ctx* ctx) {
  if (ctx) ctx->launches = 0;
}

pi_status pi_ctx_profile_begin(pi_ctx* ctx) {
  PI_ENTER(ctx);
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->prof_on = true;
  ctx->prof_used = 0;
  ctx->prof_class.clear();
  return PI_OK;
}

pi_status pi_ctx_profile_end(pi_ctx* ctx, double* ms_out, uint64_t* launches_out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, ms_out && launches_out, "null pointer");
  ctx->prof_on = false;
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (int c = 0; c < PI_PROF_CLASSES; ++c) {
    ms_out[c] = 0.0;
    launches_out[c] = 0;
  }
  for (size_t i = 0; i < ctx->prof_used; ++i) {
    float ms = 0.f;
    PI_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->prof_events[2 * i], ctx->prof_events[2 * i + 1]));
    ms_out[ctx->prof_class[i]] += ms;
    launches_out[ctx->prof_class[i]] += 1;
  }
  ctx->prof_used = 0;
  return PI_OK;
}

pi_status pi_ctx_set_option(pi_ctx* ctx, int option, int value) {
  PI_ENTER(ctx);
  switch (option) {
    case PI_OPT_TENSOR_GEMM: ctx->opt_tensor_gemm = value != 0; return PI_OK;
    case PI_OPT_CUDA_GRAPH: ctx->opt_graph = value != 0; return PI_OK;
    case PI_OPT_PDL: ctx->opt_pdl = value != 0; return PI_OK;
    case PI_OPT_ATTN_TMA: ctx->opt_attn_tma = value; return PI_OK;
    case PI_OPT_ATTN_SHARED: ctx->opt_attn_shared = value; return PI_OK;
    case PI_OPT_FUSE_PLANES: ctx->opt_fuse_planes = value != 0; return PI_OK;
    case PI_OPT_TP_PUSH: ctx->opt_tp_push = value != 0; return PI_OK;
    case PI_OPT_ATTN_FLAT:
      if (value < 0 || value > 2) return pi_fail(ctx, PI_ERR_INVALID_ARG, "PI_OPT_ATTN_FLAT is 0, 1 or 2");
      ctx->opt_attn_flat = value;
      return PI_OK;
    case PI_OPT_PEER_SPIN_LIMIT:
      PI_REQUIRE(ctx, value >= 0, "the spin limit cannot be negative");
      ctx->peer_spin_limit = (uint32_t)value;
      return PI_OK;
    case PI_OPT_GEMV_MAX_M:
      PI_REQUIRE(ctx, value >= 1, "gemv max M must be at least 1");
      ctx->opt_gemv_max_m = value;
      return PI_OK;
    default: return pi_fail(ctx, PI_ERR_INVALID_ARG, "unknown option %d", option);
  }
}

// ---- quantiser -------------------------------------------------------------------------

pi_status pi_quantize_rows_i8_dev(pi_ctx* ctx, const float* w_dev, size_t rows, size_t cols, int8_t* q_dev_out,
                                  float* scales_dev_out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, w_dev && q_dev_out && scales_dev_out, "null pointer");
  return pi_launch_quantize(ctx, w_dev, cols, rows, cols, q_dev_out, cols, scales_dev_out);
}

pi_status pi_quantize_rows_i8(pi_ctx* ctx, const float* w_host, size_t rows, size_t cols, int8_t* q_host_out,
                              float* scales_host_out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, w_host && q_host_out && scales_host_out, "null pointer");
  if (rows == 0 || cols == 0) {
    for (size_t r = 0; r < rows; ++r) scales_host_out[r] = 1.0f;
    return PI_OK;
  }
  const size_t n = rows * cols;
  PI_TRY(pi_reserve(ctx, &ctx->staging_in, n * sizeof(float)));
  PI_TRY(pi_reserve(ctx, &ctx->staging_out, n + rows * sizeof(float) + 16));
  float* w = static_cast<float*>(ctx->staging_in.ptr);
  float* sc = static_cast<float*>(ctx->staging_out.ptr);
  int8_t* q = reinterpret_cast<int8_t*>(sc + rows);
  PI_CUDA(ctx, cudaMemcpyAsync(w, w_host, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  PI_TRY(pi_launch_quantize(ctx, w, cols, rows, cols, q, cols, sc));
  PI_CUDA(ctx, cudaMemcpyAsync(q_host_out, q, n, cudaMemcpyDeviceToHost, ctx->stream));
  PI_CUDA(ctx, cudaMemcpyAsync(scales_host_out, sc, rows * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return PI_OK;
}

// ---- projections -------------------------------------------------------------------------

}  // extern "C"

static size_t elem_size(int kind) { return kind == PI_INT8 ? 1 : kind == PI_BF16 ? 2 : 4; }

pi_status pi_linear_alloc(pi_ctx* ctx, int kind, size_t full_rows, size_t full_cols, pi_split split, pi_linear** out) {
  PI_REQUIRE(ctx, out != nullptr, "out is NULL");
  *out = nullptr;
  PI_REQUIRE(ctx, kind == PI_F32 || kind == PI_INT8 || kind == PI_BF16, "unknown weight kind %d", kind);
  PI_REQUIRE(ctx, full_rows > 0 && full_cols > 0, "empty projection %zux%zu", full_rows, full_cols);
  PI_REQUIRE(ctx, full_rows < (1u << 30) && full_cols < (1u << 30), "projection too large");
  size_t rows = full_rows, cols = full_cols;
  if (ctx->tp > 1 && split == PI_SPLIT_COLUMN) {
    PI_REQUIRE(ctx, full_rows % ctx->tp == 0, "%zu rows do not split over %d ranks", full_rows, ctx->tp);
    rows = full_rows / ctx->tp;
  } else if (ctx->tp > 1 && split == PI_SPLIT_ROW) {
    PI_REQUIRE(ctx, full_cols % ctx->tp == 0, "%zu columns do not split over %d ranks", full_cols, ctx->tp);
    cols = full_cols / ctx->tp;
  }
  pi_linear* lin = new (std::nothrow) pi_linear();
  if (!lin) return pi_fail(ctx, PI_ERR_OOM, "host allocation failed");
  lin->kind = kind;
  lin->split = split;
  lin->full_rows = full_rows;
  lin->full_cols = full_cols;
  lin->rows = rows;
  lin->cols = cols;
  const size_t per16 = 16 / elem_size(kind);
  lin->ld = (cols + per16 - 1) / per16 * per16;
  cudaError_t e = cudaMalloc(&lin->w, rows * lin->ld * elem_size(kind));
  if (e == cudaSuccess && kind == PI_INT8) e = cudaMalloc(&lin->scales, rows * sizeof(float));
  if (e != cudaSuccess) {
    pi_linear_destroy(lin);
    return pi_fail(ctx, PI_ERR_OOM, "allocating a %zux%zu projection: %s", rows, cols, cudaGetErrorString(e));
  }
  *out = lin;
  return PI_OK;
}

// First row / column of this rank's shard within the full matrix.
static void shard_origin(const pi_ctx* ctx, const pi_linear* lin, size_t* r0, size_t* c0) {
  *r0 = (ctx->tp > 1 && lin->split == PI_SPLIT_COLUMN) ? (size_t)ctx->rank * lin->rows : 0;
  *c0 = (ctx->tp > 1 && lin->split == PI_SPLIT_ROW) ? (size_t)ctx->rank * lin->cols : 0;
}

// src is the FULL [full_rows x full_cols] matrix (row stride src_ld elements); the local shard is cut out.
pi_status pi_linear_fill(pi_ctx* ctx, pi_linear* lin, const void* src, size_t src_ld, bool src_on_device) {
  const size_t es = elem_size(lin->kind);
  size_t r0, c0;
  shard_origin(ctx, lin, &r0, &c0);
  const char* s = static_cast<const char*>(src) + (r0 * src_ld + c0) * es;
  if (lin->ld != lin->cols) PI_CUDA(ctx, cudaMemsetAsync(lin->w, 0, lin->rows * lin->ld * es, ctx->stream));
  PI_CUDA(ctx, cudaMemcpy2DAsync(lin->w, lin->ld * es, s, src_ld * es, lin->cols * es, lin->rows,
                                 src_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, ctx->stream));
  return PI_OK;
}

extern "C" {

pi_status pi_linear_create_i8(pi_ctx* ctx, size_t rows, size_t cols, const int8_t* q_host, const float* scales_host,
                              pi_split split, pi_linear** out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, q_host && scales_host, "null pointer");
  PI_TRY(pi_linear_alloc(ctx, PI_INT8, rows, cols, split, out));
  pi_linear* lin = *out;
  size_t r0, c0;
  shard_origin(ctx, lin, &r0, &c0);
  pi_status s = pi_linear_fill(ctx, lin, q_host, cols, false);
  if (s == PI_OK) {
    cudaError_t e = cudaMemcpyAsync(lin->scales, scales_host + r0, lin->rows * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) s = pi_fail(ctx, PI_ERR_CUDA, "uploading scales: %s", cudaGetErrorString(e));
  }
  if (s != PI_OK) {
    pi_linear_destroy(lin);
    *out = nullptr;
  }
  return s;
}

pi_status pi_linear_create_quantized(pi_ctx* ctx, size_t rows, size_t cols, const float* w_host, pi_split split,
                                     pi_linear** out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, w_host, "null pointer");
  PI_TRY(pi_linear_alloc(ctx, PI_INT8, rows, cols, split, out));
  pi_linear* lin = *out;
  // Quantise FULL rows first, then keep this rank's slice, so a row-split shard
  // carries the same codes and whole-row scales as the unsharded matrix.
  size_t r0, c0;
  shard_origin(ctx, lin, &r0, &c0);
  const size_t n = lin->rows * cols;
  pi_status s = pi_reserve(ctx, &ctx->staging_in, n * sizeof(float));
  if (s == PI_OK) s = pi_reserve(ctx, &ctx->staging_out, n);
  if (s == PI_OK) {
    float* w = static_cast<float*>(ctx->staging_in.ptr);
    int8_t* q = static_cast<int8_t*>(ctx->staging_out.ptr);
    cudaError_t e = cudaMemcpyAsync(w, w_host + r0 * cols, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) s = pi_fail(ctx, PI_ERR_CUDA, "uploading weights: %s", cudaGetErrorString(e));
    if (s == PI_OK) s = pi_launch_quantize(ctx, w, cols, lin->rows, cols, q, cols, lin->scales);
    if (s == PI_OK) {
      if (lin->ld != lin->cols) cudaMemsetAsync(lin->w, 0, lin->rows * lin->ld, ctx->stream);
      e = cudaMemcpy2DAsync(lin->w, lin->ld, q + c0, cols, lin->cols, lin->rows, cudaMemcpyDeviceToDevice, ctx->stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
      if (e != cudaSuccess) s = pi_fail(ctx, PI_ERR_CUDA, "packing codes: %s", cudaGetErrorString(e));
    }
  }
  if (s != PI_OK) {
    pi_linear_destroy(lin);
    *out = nullptr;
  }
  return s;
}

static pi_status create_plain(pi_ctx* ctx, int kind, size_t rows, size_t cols, const void* host, pi_split split,
                              pi_linear** out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, host, "null pointer");
  PI_TRY(pi_linear_alloc(ctx, kind, rows, cols, split, out));
  pi_status s = pi_linear_fill(ctx, *out, host, cols, false);
  if (s == PI_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) s = pi_fail(ctx, PI_ERR_CUDA, "upload failed");
  if (s != PI_OK) {
    pi_linear_destroy(*out);
    *out = nullptr;
  }
  return s;
}

pi_status pi_linear_create_bf16(pi_ctx* ctx, size_t rows, size_t cols, const uint16_t* w, pi_split split, pi_linear** out) {
  return create_plain(ctx, PI_BF16, rows, cols, w, split, out);
}
pi_status pi_linear_create_f32(pi_ctx* ctx, size_t rows, size_t cols, const float* w, pi_split split, pi_linear** out) {
  return create_plain(ctx, PI_F32, rows, cols, w, split, out);
}

void pi_linear_destroy(pi_linear* lin) {
  if (!lin) return;
  if (lin->owns) {
    if (lin->w) cudaFree(lin->w);
    if (lin->scales) cudaFree(lin->scales);
  }
  delete lin;
}

size_t pi_linear_rows(const pi_linear* lin) { return lin ? lin->full_rows : 0; }
size_t pi_linear_cols(const pi_linear* lin) { return lin ? lin->full_cols : 0; }
int pi_linear_kind(const pi_linear* lin) { return lin ? lin->kind : -1; }
size_t pi_linear_weight_bytes(const pi_linear* lin) {
  if (!lin) return 0;
  return lin->rows * lin->cols * elem_size(lin->kind) + (lin->kind == PI_INT8 ? lin->rows * sizeof(float) : 0);
}

pi_status pi_linear_read_i8(pi_ctx* ctx, const pi_linear* lin, int8_t* q_host_out, float* scales_host_out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, lin && lin->kind == PI_INT8, "not an int8 projection");
  if (q_host_out)
    PI_CUDA(ctx, cudaMemcpy2DAsync(q_host_out, lin->cols, lin->w, lin->ld, lin->cols, lin->rows, cudaMemcpyDeviceToHost, ctx->stream));
  if (scales_host_out)
    PI_CUDA(ctx, cudaMemcpyAsync(scales_host_out, lin->scales, lin->rows * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return PI_OK;
}

}  // extern "C"

pi_status pi_linear_forward(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a) {
  if (ctx->opt_tensor_gemm && a.M > ctx->opt_gemv_max_m && pi_gemm_tc_supported(ctx, lin, a)) return pi_launch_gemm_tc(ctx, lin, a);
  return pi_launch_gemv(ctx, lin, a);
}

extern "C" {

pi_status pi_linear_apply(pi_ctx* ctx, const pi_linear* lin, const float* x_dev, float* out_dev, int M) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, lin && x_dev && out_dev, "null pointer");
  PI_REQUIRE(ctx, M >= 1, "batch must be at least 1, got %d", M);
  pi_linear_args a;
  a.x = x_dev;
  a.x_stride = lin->cols;
  a.out = out_dev;
  a.out_stride = lin->rows;
  a.M = M;
  return pi_linear_forward(ctx, lin, a);
}

pi_status pi_linear_apply_host(pi_ctx* ctx, const pi_linear* lin, const float* x_host, float* out_host, int M) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, lin && x_host && out_host, "null pointer");
  PI_REQUIRE(ctx, M >= 1, "batch must be at least 1, got %d", M);
  const size_t xin = (size_t)M * lin->cols * sizeof(float), xout = (size_t)M * lin->rows * sizeof(float);
  PI_TRY(pi_reserve(ctx, &ctx->staging_in, xin));
  PI_TRY(pi_reserve(ctx, &ctx->staging_out, xout));
  PI_CUDA(ctx, cudaMemcpyAsync(ctx->staging_in.ptr, x_host, xin, cudaMemcpyHostToDevice, ctx->stream));
  PI_TRY(pi_linear_apply(ctx, lin, static_cast<const float*>(ctx->staging_in.ptr), static_cast<float*>(ctx->staging_out.ptr), M));
  PI_CUDA(ctx, cudaMemcpyAsync(out_host, ctx->staging_out.ptr, xout, cudaMemcpyDeviceToHost, ctx->stream));
  return pi_ctx_synchronize(ctx);
}

// ---- KV pool ---------------------------------------------------------------------------------

pi_status pi_kv_pool_create(pi_ctx* ctx, const pi_kv_layout* layout, pi_kv_pool** out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, layout && out, "null pointer");
  *out = nullptr;
  PI_REQUIRE(ctx, layout->num_layers > 0 && layout->num_blocks > 0 && layout->block_size > 0 &&
                      layout->num_kv_heads > 0 && layout->head_dim > 0,
             "KV layout fields must be positive");
  pi_kv_pool* pool = new (std::nothrow) pi_kv_pool();
  if (!pool) return pi_fail(ctx, PI_ERR_OOM, "host allocation failed");
  pool->L = *layout;
  pool->floats = (size_t)layout->num_layers * layout->num_blocks * pool->block_stride();
  cudaError_t e = cudaMalloc(&pool->data, pool->floats * sizeof(float));
  if (e != cudaSuccess) {
    delete pool;
    return pi_fail(ctx, PI_ERR_OOM, "allocating a %.2f GiB KV pool: %s", pool->floats * 4.0 / (1 << 30), cudaGetErrorString(e));
  }
  *out = pool;
  return PI_OK;
}

void pi_kv_pool_destroy(pi_kv_pool* pool) {
  if (!pool) return;
  if (pool->data) cudaFree(pool->data);
  delete pool;
}

size_t pi_kv_pool_bytes(const pi_kv_pool* pool) { return pool ? pool->floats * sizeof(float) : 0; }

pi_status pi_kv_copy_block(pi_ctx* ctx, pi_kv_pool* pool, int32_t src, int32_t dst) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, pool, "null pool");
  PI_REQUIRE(ctx, src != dst, "copy_block called with src == dst");
  PI_REQUIRE(ctx, src >= 0 && src < pool->L.num_blocks && dst >= 0 && dst < pool->L.num_blocks,
             "block %d -> %d outside the pool's %d blocks", src, dst, pool->L.num_blocks);
  return pi_launch_copy_block(ctx, pool, src, dst);
}

pi_status pi_kv_fill_normal(pi_ctx* ctx, pi_kv_pool* pool, uint64_t seed, float std) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, pool, "null pool");
  PI_TRY(pi_launch_fill_normal(ctx, pool->data, pool->floats, seed, 0xCAC4Eull, 0, std));
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return PI_OK;
}

pi_status pi_kv_upload(pi_ctx* ctx, pi_kv_pool* pool, const float* cache_host) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, pool && cache_host, "null pointer");
  PI_TRY(pi_reserve(ctx, &ctx->staging_in, pool->floats * sizeof(float)));
  PI_CUDA(ctx, cudaMemcpyAsync(ctx->staging_in.ptr, cache_host, pool->floats * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  PI_TRY(pi_launch_kv_relayout(ctx, pool, static_cast<float*>(ctx->staging_in.ptr), false));
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return PI_OK;
}

pi_status pi_kv_download(pi_ctx* ctx, const pi_kv_pool* pool, float* cache_host_out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, pool && cache_host_out, "null pointer");
  PI_TRY(pi_reserve(ctx, &ctx->staging_out, pool->floats * sizeof(float)));
  PI_TRY(pi_launch_kv_relayout(ctx, pool, static_cast<float*>(ctx->staging_out.ptr), true));
  PI_CUDA(ctx, cudaMemcpyAsync(cache_host_out, ctx->staging_out.ptr, pool->floats * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return PI_OK;
}

static pi_status kv_token_io(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int32_t block, int tok, float* k, float* v,
                             bool write) {
  PI_REQUIRE(ctx, pool && k && v, "null pointer");
  const pi_kv_layout& L = pool->L;
  PI_REQUIRE(ctx, layer >= 0 && layer < L.num_layers && block >= 0 && block < L.num_blocks && tok >= 0 && tok < L.block_size,
             "KV address (layer %d, block %d, token %d) out of range", layer, block, tok);
  for (int h = 0; h < L.num_kv_heads; ++h) {
    float* dk = pool->data + pi_kv_tile_offset(L, layer, block, h, 0) + (size_t)tok * L.head_dim;
    float* dv = pool->data + pi_kv_tile_offset(L, layer, block, h, 1) + (size_t)tok * L.head_dim;
    const size_t bytes = L.head_dim * sizeof(float);
    if (write) {
      PI_CUDA(ctx, cudaMemcpyAsync(dk, k + (size_t)h * L.head_dim, bytes, cudaMemcpyHostToDevice, ctx->stream));
      PI_CUDA(ctx, cudaMemcpyAsync(dv, v + (size_t)h * L.head_dim, bytes, cudaMemcpyHostToDevice, ctx->stream));
    } else {
      PI_CUDA(ctx, cudaMemcpyAsync(k + (size_t)h * L.head_dim, dk, bytes, cudaMemcpyDeviceToHost, ctx->stream));
      PI_CUDA(ctx, cudaMemcpyAsync(v + (size_t)h * L.head_dim, dv, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    }
  }
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return PI_OK;
}

pi_status pi_kv_write_token(pi_ctx* ctx, pi_kv_pool* pool, int layer, int32_t block, int tok, const float* k_host,
                            const float* v_host) {
  PI_ENTER(ctx);
  return kv_token_io(ctx, pool, layer, block, tok, const_cast<float*>(k_host), const_cast<float*>(v_host), true);
}
pi_status pi_kv_read_token(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int32_t block, int tok, float* k_host_out,
                           float* v_host_out) {
  PI_ENTER(ctx);
  return kv_token_io(ctx, pool, layer, block, tok, k_host_out, v_host_out, false);
}

// ---- paged attention -----------------------------------------------------------------------------

static pi_status check_tables(pi_ctx* ctx, const pi_kv_pool* pool, const int32_t* tables, int max_blocks,
                              const int32_t* lens, int B) {
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < lens[b] && i < max_blocks; ++i) {
      const int32_t pb = tables[(size_t)b * max_blocks + i];
      PI_REQUIRE(ctx, pb >= 0 && pb < pool->L.num_blocks, "entry %d maps logical block %d to physical block %d of %d", b, i,
                 pb, pool->L.num_blocks);
    }
  return PI_OK;
}

pi_status pi_paged_attention(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q_dev,
                             size_t q_stride, float* out_dev, size_t out_stride, const int32_t* block_tables_host,
                             int max_blocks, const int32_t* table_lens_host, const int32_t* pos_host,
                             const int32_t* start_host, int B) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, pool && q_dev && out_dev && table_lens_host && pos_host && start_host, "null pointer");
  PI_REQUIRE(ctx, block_tables_host || max_blocks == 0, "null block tables");
  if (B == 0) return PI_OK;
  PI_REQUIRE(ctx, B > 0, "negative batch");
  PI_TRY(check_tables(ctx, pool, block_tables_host, max_blocks, table_lens_host, B));
  pi_attn_batch batch;
  PI_TRY(pi_upload_attn_batch(ctx, block_tables_host, max_blocks, table_lens_host, pos_host, start_host, B,
                              pool->L.block_size, pool->L.num_blocks, &batch));
  if (ctx->opt_attn_flat >= 2) PI_TRY(pi_attention_prepare(ctx, pool, num_heads, batch));
  return pi_launch_attention(ctx, pool, layer, num_heads, q_dev, q_stride, out_dev, out_stride, batch);
}

pi_status pi_paged_attention_host(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q_host,
                                  float* out_host, const int32_t* block_tables_host, int max_blocks,
                                  const int32_t* table_lens_host, const int32_t* pos_host, const int32_t* start_host,
                                  int B) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, pool && q_host && out_host, "null pointer");
  if (B == 0) return PI_OK;
  PI_REQUIRE(ctx, B > 0 && num_heads > 0, "bad batch / head count");
  const size_t row = (size_t)num_heads * pool->L.head_dim, bytes = (size_t)B * row * sizeof(float);
  PI_TRY(pi_reserve(ctx, &ctx->staging_in, bytes));
  PI_TRY(pi_reserve(ctx, &ctx->staging_out, bytes));
  PI_CUDA(ctx, cudaMemcpyAsync(ctx->staging_in.ptr, q_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  PI_TRY(pi_paged_attention(ctx, pool, layer, num_heads, static_cast<const float*>(ctx->staging_in.ptr), row,
                            static_cast<float*>(ctx->staging_out.ptr), row, block_tables_host, max_blocks,
                            table_lens_host, pos_host, start_host, B));
  PI_CUDA(ctx, cudaMemcpyAsync(out_host, ctx->staging_out.ptr, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return pi_ctx_synchronize(ctx);
}

// ---- glue with host buffers --------------------------------------------------------------------------

pi_status pi_rms_norm_host(pi_ctx* ctx, float* x_host_inout, const float* weight_host, int rows, int n, float eps) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, x_host_inout && weight_host && rows >= 0 && n > 0, "bad arguments");
  if (rows == 0) return PI_OK;
  const size_t xb = (size_t)rows * n * sizeof(float), wb = (size_t)n * sizeof(float);
  PI_TRY(pi_reserve(ctx, &ctx->staging_in, xb + wb));
  float* x = static_cast<float*>(ctx->staging_in.ptr);
  float* w = x + (size_t)rows * n;
  PI_CUDA(ctx, cudaMemcpyAsync(x, x_host_inout, xb, cudaMemcpyHostToDevice, ctx->stream));
  PI_CUDA(ctx, cudaMemcpyAsync(w, weight_host, wb, cudaMemcpyHostToDevice, ctx->stream));
  PI_TRY(pi_launch_rms_norm(ctx, x, n, w, rows, n, eps));
  PI_CUDA(ctx, cudaMemcpyAsync(x_host_inout, x, xb, cudaMemcpyDeviceToHost, ctx->stream));
  return pi_ctx_synchronize(ctx);
}

pi_status pi_rope_host(pi_ctx* ctx, float* x_host_inout, const int32_t* pos_host, int rows, int heads, int head_dim,
                       float theta, int style) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, x_host_inout && pos_host && rows >= 0 && heads > 0 && head_dim > 0, "bad arguments");
  PI_REQUIRE(ctx, style == 0 || style == 1, "rope style must be 0 (NeoX) or 1 (interleaved)");
  if (rows == 0) return PI_OK;
  const int half = head_dim / 2;
  // The table is built on the host with the host libm, row r holding the angles of pos[r].
  std::vector<float> table((size_t)rows * half * 2);
  std::vector<int32_t> ridx(rows);
  for (int r = 0; r < rows; ++r) {
    PI_REQUIRE(ctx, pos_host[r] >= 0, "negative position");
    pi_host_rope_table(pos_host[r], head_dim, theta, &table[(size_t)r * half], &table[(size_t)(rows + r) * half]);
    ridx[r] = r;
  }
  const size_t xb = (size_t)rows * heads * head_dim * sizeof(float), tb = table.size() * sizeof(float), ib = rows * sizeof(int32_t);
  PI_TRY(pi_reserve(ctx, &ctx->staging_in, xb + tb + ib + 64));
  float* x = static_cast<float*>(ctx->staging_in.ptr);
  float* t = x + (size_t)rows * heads * head_dim;
  int32_t* idx = reinterpret_cast<int32_t*>(t + table.size());
  PI_CUDA(ctx, cudaMemcpyAsync(x, x_host_inout, xb, cudaMemcpyHostToDevice, ctx->stream));
  PI_CUDA(ctx, cudaMemcpyAsync(t, table.data(), tb, cudaMemcpyHostToDevice, ctx->stream));
  PI_CUDA(ctx, cudaMemcpyAsync(idx, ridx.data(), ib, cudaMemcpyHostToDevice, ctx->stream));
  PI_TRY(pi_launch_rope(ctx, x, (size_t)heads * head_dim, heads, head_dim, idx, t, t + (size_t)rows * half, style, rows));
  PI_CUDA(ctx, cudaMemcpyAsync(x_host_inout, x, xb, cudaMemcpyDeviceToHost, ctx->stream));
  return pi_ctx_synchronize(ctx);
}

pi_status pi_swiglu_host(pi_ctx* ctx, float* gate_host_inout, const float* up_host, size_t n) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, gate_host_inout && up_host, "null pointer");
  if (n == 0) return PI_OK;
  PI_TRY(pi_reserve(ctx, &ctx->staging_in, 2 * n * sizeof(float)));
  float* g = static_cast<float*>(ctx->staging_in.ptr);
  PI_CUDA(ctx, cudaMemcpyAsync(g, gate_host_inout, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  PI_CUDA(ctx, cudaMemcpyAsync(g + n, up_host, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  PI_TRY(pi_launch_swiglu(ctx, g, g + n, n));
  PI_CUDA(ctx, cudaMemcpyAsync(gate_host_inout, g, n * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  return pi_ctx_synchronize(ctx);
}

pi_status pi_argmax_host(pi_ctx* ctx, const float* logits_host, int rows, int n, uint32_t* out_host) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, logits_host && out_host && rows >= 0 && n > 0, "bad arguments");
  if (rows == 0) return PI_OK;
  const size_t lb = (size_t)rows * n * sizeof(float);
  PI_TRY(pi_reserve(ctx, &ctx->staging_in, lb));
  PI_TRY(pi_reserve(ctx, &ctx->staging_out, rows * sizeof(uint32_t)));
  PI_CUDA(ctx, cudaMemcpyAsync(ctx->staging_in.ptr, logits_host, lb, cudaMemcpyHostToDevice, ctx->stream));
  PI_TRY(pi_launch_argmax(ctx, static_cast<const float*>(ctx->staging_in.ptr), n, rows, n, static_cast<uint32_t*>(ctx->staging_out.ptr)));
  PI_CUDA(ctx, cudaMemcpyAsync(out_host, ctx->staging_out.ptr, rows * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  return pi_ctx_synchronize(ctx);
}

}  // extern "C"
