// Per-token glue kernels between the projections and attention: embedding
// gather, RMSNorm, rotary embedding fused with the K/V scatter into the paged
// pool, SwiGLU, residual add, greedy argmax, copy-on-write block copy, and the
// pool re-layout used by upload/download.
//
// Replaces (reference): bf16_bytes_into_f32 + token % vocab (src/model.rs:457-462,
// :1015-1020), math::rms_norm (src/math.rs:4-22), rope_rotate (:344-367) and the
// K/V scatter (src/model.rs:1065-1107), swiglu (src/math.rs:292-302), residual
// adds (src/model.rs:1127-1129), sampling::argmax (src/sampling.rs:140-147),
// KvLayout::copy_block (src/memory/layout.rs:82-96).
#include <math.h>

#include "pi_common.cuh"

namespace {

__global__ void embed_kernel(const uint16_t* __restrict__ table, int vocab, int hidden,
                             const uint32_t* __restrict__ tokens, float* __restrict__ x) {
  // strict: the step's attention work list (built by the kernel ahead of this one) is complete before any later kernel
  // of the step starts, so the attention kernels of layers > 0 may read it ahead of their own dependency wait
  pi_grid_dependency_wait_strict();
  const int b = blockIdx.x;
  const size_t token = (size_t)(tokens[b] % (uint32_t)vocab);
  const uint16_t* src = table + token * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) x[(size_t)b * hidden + i] = pi_bf16_bits_to_f32(src[i]);
}

__global__ void __launch_bounds__(256) rms_norm_kernel(float* __restrict__ x, size_t stride,
                                                       const float* __restrict__ weight, int n, float eps) {
  __shared__ float red[8];
  __shared__ float s_inv;
  float* row = x + (size_t)blockIdx.x * stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  ss = pi_warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    s_inv = 1.0f / sqrtf(t / (float)n + eps);
  }
  __syncthreads();
  const float inv = s_inv;
  for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = row[i] * inv * weight[i];
}

__device__ __forceinline__ void rotate_pair(float& a, float& b, float c, float s) {
  const float na = a * c - b * s;
  const float nb = b * c + a * s;
  a = na;
  b = nb;
}

// One CTA per (entry, head slot).  Slots [0, H) rotate a query head in place;
// slots [H, H+KH) rotate a key head and scatter it with its value head into the
// pool; a position whose logical block is unmapped is skipped silently.
__global__ void rope_kv_write_kernel(float* __restrict__ qkv, size_t qkv_stride, int H, int KH, int hd,
                                     const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, int style,
                                     float* __restrict__ kv, pi_kv_layout L, int layer,
                                     const int32_t* __restrict__ tables, int max_blocks,
                                     const int32_t* __restrict__ lens, const int32_t* __restrict__ pos) {
  pi_grid_dependency_wait();
  const int b = blockIdx.y, slot = blockIdx.x, half = hd >> 1;
  const int p = pos[b];
  const float* cs = rope_cos + (size_t)p * half;
  const float* sn = rope_sin + (size_t)p * half;
  float* row = qkv + (size_t)b * qkv_stride;
  if (slot < H) {
    float* v = row + (size_t)slot * hd;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      const int ia = style == 0 ? j : 2 * j, ib = style == 0 ? j + half : 2 * j + 1;
      float a = v[ia], c = v[ib];
      rotate_pair(a, c, cs[j], sn[j]);
      v[ia] = a;
      v[ib] = c;
    }
    return;
  }
  const int kh = slot - H;
  float* kvec = row + (size_t)(H + kh) * hd;
  const float* vvec = row + (size_t)(H + KH + kh) * hd;
  const int lb = p / L.block_size, off = p % L.block_size;
  const bool mapped = lb < lens[b];
  const int pb = mapped ? tables[(size_t)b * max_blocks + lb] : 0;
  float* kdst = kv + pi_kv_tile_offset(L, layer, pb, kh, 0) + (size_t)off * hd;
  float* vdst = kv + pi_kv_tile_offset(L, layer, pb, kh, 1) + (size_t)off * hd;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const int ia = style == 0 ? j : 2 * j, ib = style == 0 ? j + half : 2 * j + 1;
    float a = kvec[ia], c = kvec[ib];
    rotate_pair(a, c, cs[j], sn[j]);
    kvec[ia] = a;
    kvec[ib] = c;
    if (mapped) {
      kdst[ia] = a;
      kdst[ib] = c;
      vdst[ia] = vvec[ia];
      vdst[ib] = vvec[ib];
    }
  }
  if (mapped && (hd & 1) && threadIdx.x == 0) {  // odd head_dim: the last element is not rotated
    kdst[hd - 1] = kvec[hd - 1];
    vdst[hd - 1] = vvec[hd - 1];
  }
}

__global__ void rope_kernel(float* __restrict__ x, size_t stride, int heads, int hd, const int32_t* __restrict__ pos,
                            const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, int style) {
  const int r = blockIdx.y, h = blockIdx.x, half = hd >> 1;
  const float* cs = rope_cos + (size_t)pos[r] * half;
  const float* sn = rope_sin + (size_t)pos[r] * half;
  float* v = x + (size_t)r * stride + (size_t)h * hd;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const int ia = style == 0 ? j : 2 * j, ib = style == 0 ? j + half : 2 * j + 1;
    float a = v[ia], c = v[ib];
    rotate_pair(a, c, cs[j], sn[j]);
    v[ia] = a;
    v[ib] = c;
  }
}

__global__ void swiglu_kernel(float* __restrict__ gate, const float* __restrict__ up, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float g = gate[i];
    gate[i] = (g / (1.0f + expf(-g))) * up[i];
  }
}

__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
  pi_grid_dependency_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] += y[i];
}

// f32::total_cmp as a signed integer key.
__device__ __forceinline__ int total_order_key(float f) {
  const int b = __float_as_int(f);
  return b ^ (int)(((unsigned)(b >> 31)) >> 1);
}
__device__ __forceinline__ void argmax_merge(int& bk, int& bi, int k, int i) {
  if (k > bk || (k == bk && i > bi)) {
    bk = k;
    bi = i;
  }
}

__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, size_t stride, int n,
                                                      uint32_t* __restrict__ out) {
  pi_grid_dependency_wait();
  __shared__ int sk[32], si[32];
  const float* row = logits + (size_t)blockIdx.x * stride;
  int bk = INT_MIN, bi = -1;
  if ((((uintptr_t)row) & 15) == 0) {
    // four independent candidates per thread over 16-byte loads, merged in index order afterwards
    int k4[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN}, i4[4] = {-1, -1, -1, -1};
    const int n4 = n >> 2;
    for (int v = threadIdx.x; v < n4; v += blockDim.x) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(row) + v);
      argmax_merge(k4[0], i4[0], total_order_key(f.x), 4 * v);
      argmax_merge(k4[1], i4[1], total_order_key(f.y), 4 * v + 1);
      argmax_merge(k4[2], i4[2], total_order_key(f.z), 4 * v + 2);
      argmax_merge(k4[3], i4[3], total_order_key(f.w), 4 * v + 3);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) argmax_merge(bk, bi, k4[j], i4[j]);
    for (int i = 4 * n4 + threadIdx.x; i < n; i += blockDim.x) argmax_merge(bk, bi, total_order_key(row[i]), i);
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) argmax_merge(bk, bi, total_order_key(row[i]), i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const int k = __shfl_xor_sync(0xffffffffu, bk, o), i = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_merge(bk, bi, k, i);
  }
  if ((threadIdx.x & 31) == 0) {
    sk[threadIdx.x >> 5] = bk;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) argmax_merge(bk, bi, sk[w], si[w]);
    out[blockIdx.x] = bi < 0 ? 0u : (uint32_t)bi;
  }
}

// grid (chunks, layers): copy one physical block's span in every layer.
__global__ void copy_block_kernel(float* __restrict__ kv, size_t layer_stride, size_t block_stride, int src, int dst) {
  const float* sp = kv + (size_t)blockIdx.y * layer_stride + (size_t)src * block_stride;
  float* dp = kv + (size_t)blockIdx.y * layer_stride + (size_t)dst * block_stride;
  if ((block_stride & 3) == 0) {  // every span then starts on a 16-byte boundary
    const float4* s = reinterpret_cast<const float4*>(sp);
    float4* d = reinterpret_cast<float4*>(dp);
    const size_t n4 = block_stride / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) d[i] = s[i];
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < block_stride; i += (size_t)gridDim.x * blockDim.x)
      dp[i] = sp[i];
  }
}

// Between the reference layout [layer][block][tok][kvh][k|v][hd] and the device
// layout [layer][block][kvh][k|v][tok][hd].
__global__ void kv_relayout_kernel(float* __restrict__ dev, float* __restrict__ ref, pi_kv_layout L, size_t total,
                                   int to_reference) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i;  // index in the reference layout
    const int d = (int)(r % L.head_dim);
    r /= L.head_dim;
    const int isv = (int)(r & 1);
    r >>= 1;
    const int kh = (int)(r % L.num_kv_heads);
    r /= L.num_kv_heads;
    const int tok = (int)(r % L.block_size);
    r /= L.block_size;  // r = layer*num_blocks + block
    const size_t j = (((r * L.num_kv_heads + kh) * 2 + isv) * L.block_size + tok) * L.head_dim + d;
    if (to_reference) ref[i] = dev[j];
    else dev[j] = ref[i];
  }
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Two normals per counter via Box-Muller on 24-bit uniforms.
__global__ void fill_normal_kernel(float* __restrict__ out, size_t n, uint64_t seed, uint64_t stream_id,
                                   uint64_t pair_offset, float std) {
  const uint64_t key = splitmix64(seed ^ splitmix64(stream_id)) + pair_offset;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i * 2 < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t r = splitmix64(key + i);
    const float u1 = ((float)((r >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f);
    const float u2 = (float)((r >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
    const float rad = sqrtf(-2.0f * logf(u1));
    float s, c;
    sincospif(2.0f * u2, &s, &c);
    out[2 * i] = std * rad * c;
    if (2 * i + 1 < n) out[2 * i + 1] = std * rad * s;
  }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, uint16_t* __restrict__ out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t u = __float_as_uint(in[i]);
    out[i] = (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);  // round to nearest even
  }
}

__global__ void bf16_to_f32_kernel(const uint16_t* __restrict__ in, size_t in_ld, float* __restrict__ out,
                                   size_t out_ld, size_t rows, size_t cols) {
  const size_t total = rows * cols;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols, c = i - r * cols;
    out[r * out_ld + c] = pi_bf16_bits_to_f32(in[r * in_ld + c]);
  }
}

inline unsigned grid_for(size_t n, int threads, int sm_count) {
  const size_t want = (n + threads - 1) / threads;
  const size_t cap = (size_t)sm_count * 16;
  return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(pi_ctx* ctx, void (*k)(KArgs...), dim3 grid, dim3 block, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, k, KArgs(args)...);
}

}  // namespace

#define PI_LAUNCHED(ctx, e)                                                                              \
  do {                                                                                                   \
    cudaError_t _le = (e);                                                                               \
    if (_le != cudaSuccess)                                                                              \
      return pi_fail((ctx), PI_ERR_CUDA, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(_le),   \
                     __FILE__, __LINE__);                                                                \
    (ctx)->launches++;                                                                                   \
  } while (0)

void pi_host_rope_table(int pos, int head_dim, float theta, float* cos_out, float* sin_out) {
  // reference math::rope_table (src/math.rs:331-341): all in f32 with the host libm.
  const int half = head_dim / 2;
  for (int j = 0; j < half; ++j) {
    const float freq = 1.0f / powf(theta, (float)(2 * j) / (float)head_dim);
    const float a = (float)pos * freq;
    sin_out[j] = sinf(a);
    cos_out[j] = cosf(a);
  }
}

pi_status pi_launch_embed(pi_ctx* ctx, const uint16_t* table_bf16, int vocab, int hidden, const uint32_t* tokens_dev,
                          int B, float* x) {
  pi_prof_scope prof(ctx, PI_PROF_OTHER);
  PI_LAUNCHED(ctx, launch_pdl(ctx, embed_kernel, dim3(B), dim3(256), table_bf16, vocab, hidden, tokens_dev, x));
  return PI_OK;
}

pi_status pi_launch_rms_norm(pi_ctx* ctx, float* x, size_t stride, const float* weight, int rows, int n, float eps) {
  rms_norm_kernel<<<rows, 256, 0, ctx->stream>>>(x, stride, weight, n, eps);
  PI_CHECK_LAUNCH(ctx);
  return PI_OK;
}

pi_status pi_launch_rope_kv_write(pi_ctx* ctx, float* qkv, size_t qkv_stride, int num_heads, int num_kv_heads,
                                  int head_dim, const float* rope_cos, const float* rope_sin, int style,
                                  pi_kv_pool* pool, int layer, const pi_attn_batch& batch) {
  const int threads = head_dim / 2 >= 64 ? 64 : 32;
  pi_prof_scope prof(ctx, PI_PROF_ROPE_KV);
  PI_LAUNCHED(ctx, launch_pdl(ctx, rope_kv_write_kernel, dim3(num_heads + num_kv_heads, batch.B), dim3(threads), qkv,
                              qkv_stride, num_heads, num_kv_heads, head_dim, rope_cos, rope_sin, style, pool->data,
                              pool->L, layer, batch.tables, batch.max_blocks, batch.lens, batch.pos));
  return PI_OK;
}

pi_status pi_launch_rope(pi_ctx* ctx, float* x, size_t stride, int heads, int head_dim, const int32_t* pos_dev,
                         const float* rope_cos, const float* rope_sin, int style, int rows) {
  rope_kernel<<<dim3(heads, rows), 32, 0, ctx->stream>>>(x, stride, heads, head_dim, pos_dev, rope_cos, rope_sin, style);
  PI_CHECK_LAUNCH(ctx);
  return PI_OK;
}

pi_status pi_launch_swiglu(pi_ctx* ctx, float* gate, const float* up, size_t n) {
  if (n == 0) return PI_OK;
  swiglu_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(gate, up, n);
  PI_CHECK_LAUNCH(ctx);
  return PI_OK;
}

pi_status pi_launch_add(pi_ctx* ctx, float* x, const float* y, size_t n) {
  pi_prof_scope prof(ctx, PI_PROF_OTHER);
  if (n == 0) return PI_OK;
  PI_LAUNCHED(ctx, launch_pdl(ctx, add_kernel, dim3(grid_for(n, 256, ctx->sm_count)), dim3(256), x, y, n));
  return PI_OK;
}

pi_status pi_launch_argmax(pi_ctx* ctx, const float* logits, size_t stride, int rows, int n, uint32_t* out) {
  pi_prof_scope prof(ctx, PI_PROF_OTHER);
  PI_LAUNCHED(ctx, launch_pdl(ctx, argmax_kernel, dim3(rows), dim3(1024), logits, stride, n, out));
  return PI_OK;
}

pi_status pi_launch_copy_block(pi_ctx* ctx, pi_kv_pool* pool, int src, int dst) {
  const size_t bs = pool->block_stride();
  const size_t layer_stride = bs * pool->L.num_blocks;
  unsigned chunks = (unsigned)((bs / 4 + 255) / 256);
  if (chunks < 1) chunks = 1;
  if (chunks > 64) chunks = 64;
  copy_block_kernel<<<dim3(chunks, pool->L.num_layers), 256, 0, ctx->stream>>>(pool->data, layer_stride, bs, src, dst);
  PI_CHECK_LAUNCH(ctx);
  return PI_OK;
}

pi_status pi_launch_kv_relayout(pi_ctx* ctx, const pi_kv_pool* pool, float* ref_layout, bool to_reference) {
  if (pool->floats == 0) return PI_OK;
  kv_relayout_kernel<<<grid_for(pool->floats, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
      pool->data, ref_layout, pool->L, pool->floats, to_reference ? 1 : 0);
  PI_CHECK_LAUNCH(ctx);
  return PI_OK;
}

pi_status pi_launch_fill_normal(pi_ctx* ctx, float* out, size_t n, uint64_t seed, uint64_t stream_id,
                                uint64_t pair_offset, float std) {
  if (n == 0) return PI_OK;
  fill_normal_kernel<<<grid_for((n + 1) / 2, 256, ctx->sm_count), 256, 0, ctx->stream>>>(out, n, seed, stream_id, pair_offset, std);
  PI_CHECK_LAUNCH(ctx);
  return PI_OK;
}

pi_status pi_launch_f32_to_bf16(pi_ctx* ctx, const float* in, uint16_t* out, size_t n) {
  if (n == 0) return PI_OK;
  f32_to_bf16_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(in, out, n);
  PI_CHECK_LAUNCH(ctx);
  return PI_OK;
}

pi_status pi_launch_bf16_to_f32(pi_ctx* ctx, const uint16_t* in, size_t in_ld, float* out, size_t out_ld, size_t rows,
                                size_t cols) {
  if (rows * cols == 0) return PI_OK;
  bf16_to_f32_kernel<<<grid_for(rows * cols, 256, ctx->sm_count), 256, 0, ctx->stream>>>(in, in_ld, out, out_ld, rows, cols);
  PI_CHECK_LAUNCH(ctx);
  return PI_OK;
}
