// Paged attention for entries that SHARE one block table: the positions of a prefill chunk, or the draft positions
// of a speculative verify group (reference: src/model.rs:1222-1255 feeds every position of a chunk through
// PagedAttention::run as its own entry, src/attention.rs:141-265; src/engine.rs:702-761 does the same for drafts).
//
// The decode kernel streams the whole window once per entry.  Here one CTA owns a tile of 64 query rows -
// (position, query head) pairs of ONE kv head, i.e. 64 / kv_group positions - and walks the window once for all of
// them, flash-attention style:
//
//   * K and V tiles of 64 tokens (four physical blocks, looked up in the shared table) are staged in shared memory
//     with cp.async, double buffered; rows are padded by 4 floats so that every fragment load below is free of bank
//     conflicts.  Tokens outside [lowest start, highest position] of the tile and tokens of unmapped blocks are
//     stored as zeros, never read from the pool.
//   * scores = Q K^T and out += P V run on the tensor cores with mma.sync m16n8k8 TF32, each product as THREE
//     MMAs over an exact split x = hi + lo (hi = the upper 19 bits of the f32, lo = x - hi):
//     hi*hi + lo*hi + hi*lo; the dropped lo*lo term is 2^-22 relative, so the result is f32-equivalent
//     and agrees with the decode kernel to a few 1e-6 (both use ex2.approx).
//   * softmax is online in the log2 domain, per row, in the accumulator registers; a position outside the row's
//     window [start, pos] or in an unmapped block scores -inf; an empty window gives zeros.
//   * the probabilities feed the second product straight from the score accumulators: the k index of that MMA is a
//     token, so tokens are simply visited in the order the accumulator layout holds them (2t, 2t+1 per lane).
//
// One warp = 16 rows; 4 warps per CTA; grid (kv heads, row tiles), the tiles with the longest windows first.
#include <math.h>

#include <algorithm>

#include "pi_common.cuh"

namespace {

constexpr int kRows = 64;          // query rows per CTA
constexpr int kTile = 64;          // tokens per K/V tile
constexpr int kBlock = 16;         // tokens per physical block (the only block size this kernel takes)
constexpr int kWarps = 4;
constexpr uint32_t kHiMask = 0xffffe000u;

struct SharedAttnParams {
  const float* q;
  size_t q_stride;
  float* out;
  size_t out_stride;
  const float* kv;
  pi_kv_layout L;
  int layer;
  int B;                  // entries
  const int32_t* table;   // the shared row [len]
  int len;
  const int32_t* pos;
  const int32_t* start;
  float scale2;           // 1/sqrt(head_dim) * log2(e)
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(x) & kHiMask;
  lo = __float_as_uint(x - __uint_as_float(hi));
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <int HD, int G>
__global__ void __launch_bounds__(kWarps * 32) attn_shared_table_kernel(const SharedAttnParams p) {
  constexpr int QS = HD + 4;               // padded row stride (floats)
  constexpr int PPC = kRows / G;           // positions per CTA
  constexpr int C4 = HD / 4;               // 16-byte chunks per row
  constexpr int KS = HD / 8;               // k steps of the score product = n blocks of the output product
  constexpr int NB = kTile / 8;            // n blocks of the score product = k steps of the output product
  extern __shared__ __align__(16) float smem[];
  float* q_hi = smem;                      // [64][QS]
  float* q_lo = q_hi + kRows * QS;
  float* k_s = q_lo + kRows * QS;          // [2][64][QS]
  float* v_s = k_s + 2 * kTile * QS;       // [2][64][QS]
  __shared__ int s_lo, s_hi;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  const int kvh = blockIdx.x;
  const int tile_row = (int)gridDim.y - 1 - (int)blockIdx.y;   // long windows first
  const int e0 = tile_row * PPC;

  if (tid == 0) {
    s_lo = 0x7fffffff;
    s_hi = -1;
  }
  pi_grid_dependency_wait();
  pi_grid_launch_dependents();
  __syncthreads();
  if (tid < PPC && e0 + tid < p.B) {
    const int ps = p.pos[e0 + tid], st = p.start[e0 + tid];
    if (st <= ps) {
      atomicMin(&s_lo, st);
      atomicMax(&s_hi, ps);
    }
  }

  // ---- Q: scale into the log2 domain, split, stage -------------------------------------------------------------
  for (int c = tid; c < kRows * C4; c += kWarps * 32) {
    const int r = c / C4, d4 = c - r * C4;
    const int e = e0 + r / G, h = kvh * G + r % G;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e < p.B) x = __ldg(reinterpret_cast<const float4*>(p.q + (size_t)e * p.q_stride + (size_t)h * HD + d4 * 4));
    const float xs[4] = {x.x * p.scale2, x.y * p.scale2, x.z * p.scale2, x.w * p.scale2};
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) split_tf32(xs[i], hi[i], lo[i]);
    *reinterpret_cast<uint4*>(q_hi + r * QS + d4 * 4) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<uint4*>(q_lo + r * QS + d4 * 4) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  }
  __syncthreads();
  const int t_min = s_lo, t_max = s_hi;

  // the two rows of this lane
  const int r0 = warp * 16 + gid, r1 = r0 + 8;
  const int en0 = e0 + r0 / G, en1 = e0 + r1 / G;
  int pos0 = -1, st0 = 0, pos1 = -1, st1 = 0;
  if (en0 < p.B) {
    pos0 = p.pos[en0];
    st0 = p.start[en0];
  }
  if (en1 < p.B) {
    pos1 = p.pos[en1];
    st1 = p.start[en1];
  }

  float o[KS][4];
#pragma unroll
  for (int i = 0; i < KS; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  const int jt_first = t_max >= 0 ? t_min / kTile : 0;
  const int ntiles = t_max >= 0 ? t_max / kTile - jt_first + 1 : 0;

  // physical block of logical block lb, or -1 when it is unmapped or holds nothing this tile may read
  auto block_of = [&](int lb) -> int {
    if (lb >= p.len || lb * kBlock > t_max || lb * kBlock + kBlock - 1 < t_min) return -1;
    return p.table[lb];
  };
  auto load_tile = [&](int jt, int stage) {
    float* kd = k_s + (size_t)stage * kTile * QS;
    float* vd = v_s + (size_t)stage * kTile * QS;
    int pb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pb[i] = block_of(jt * 4 + i);
    constexpr int kChunks = 4 * 2 * kBlock * C4;
#pragma unroll 4
    for (int c = tid; c < kChunks; c += kWarps * 32) {
      const int d4 = c % C4, tok = (c / C4) % kBlock, is_v = (c / (C4 * kBlock)) & 1, blk = c / (C4 * kBlock * 2);
      const int t = (jt * 4 + blk) * kBlock + tok;
      float* dst = (is_v ? vd : kd) + (blk * kBlock + tok) * QS + d4 * 4;
      const int b = blk == 0 ? pb[0] : blk == 1 ? pb[1] : blk == 2 ? pb[2] : pb[3];
      if (b >= 0 && t >= t_min && t <= t_max) {
        const float* src = p.kv + pi_kv_tile_offset(p.L, p.layer, b, kvh, is_v) + tok * HD + d4 * 4;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
      } else {
        *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  if (ntiles > 0) load_tile(jt_first, 0);
  for (int j = 0; j < ntiles; ++j) {
    const int jt = jt_first + j, stage = j & 1;
    if (j + 1 < ntiles) {
      load_tile(jt + 1, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* kt = k_s + (size_t)stage * kTile * QS;
    const float* vt = v_s + (size_t)stage * kTile * QS;

    // ---- scores: S[16 rows][64 tokens] = Q K^T ---------------------------------------------------------------
    float s[NB][4];
#pragma unroll
    for (int i = 0; i < NB; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 2
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t ah[4], al[4];
      const int qo0 = r0 * QS + ks * 8 + tig, qo1 = r1 * QS + ks * 8 + tig;
      ah[0] = __float_as_uint(q_hi[qo0]);
      ah[1] = __float_as_uint(q_hi[qo1]);
      ah[2] = __float_as_uint(q_hi[qo0 + 4]);
      ah[3] = __float_as_uint(q_hi[qo1 + 4]);
      al[0] = __float_as_uint(q_lo[qo0]);
      al[1] = __float_as_uint(q_lo[qo1]);
      al[2] = __float_as_uint(q_lo[qo0 + 4]);
      al[3] = __float_as_uint(q_lo[qo1 + 4]);
      // four n blocks at a time: consecutive MMAs go to different accumulators, so none waits for the one before it
#pragma unroll
      for (int nb0 = 0; nb0 < NB; nb0 += 4) {
        uint32_t h0[4], g0[4], h1[4], g1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float* kp = kt + ((nb0 + i) * 8 + gid) * QS + ks * 8 + tig;
          split_tf32(kp[0], h0[i], g0[i]);
          split_tf32(kp[4], h1[i], g1[i]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_tf32(s[nb0 + i], al, h0[i], h1[i]);
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_tf32(s[nb0 + i], ah, g0[i], g1[i]);
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_tf32(s[nb0 + i], ah, h0[i], h1[i]);
      }
    }

    // ---- mask + online softmax (log2 domain) --------------------------------------------------------------------
    unsigned mapped = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) mapped |= (block_of(jt * 4 + i) >= 0 ? 1u : 0u) << i;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const bool blk_ok = (mapped >> (nb >> 1)) & 1u;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int t = jt * kTile + nb * 8 + 2 * tig + c;
        if (!(blk_ok && t >= st0 && t <= pos0)) s[nb][c] = -INFINITY;
        if (!(blk_ok && t >= st1 && t <= pos1)) s[nb][2 + c] = -INFINITY;
        mx0 = fmaxf(mx0, s[nb][c]);
        mx1 = fmaxf(mx1, s[nb][2 + c]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float corr0 = (m0 == -INFINITY) ? 1.f : ex2f(m0 - mn0), corr1 = (m1 == -INFINITY) ? 1.f : ex2f(m1 - mn1);
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const float a = (s[nb][c] == -INFINITY) ? 0.f : ex2f(s[nb][c] - mn0);
        const float b = (s[nb][2 + c] == -INFINITY) ? 0.f : ex2f(s[nb][2 + c] - mn1);
        s[nb][c] = a;
        s[nb][2 + c] = b;
        ps0 += a;
        ps1 += b;
      }
    }
    l0 = l0 * corr0 + ps0;
    l1 = l1 * corr1 + ps1;
    m0 = mn0;
    m1 = mn1;
    if (__any_sync(0xffffffffu, corr0 != 1.f || corr1 != 1.f)) {
#pragma unroll
      for (int i = 0; i < KS; ++i) {
        o[i][0] *= corr0;
        o[i][1] *= corr0;
        o[i][2] *= corr1;
        o[i][3] *= corr1;
      }
    }

    // ---- out += P V: the k index runs over the tile's tokens in accumulator order ---------------------------------
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      uint32_t ah[4], al[4];
      split_tf32(s[nb][0], ah[0], al[0]);   // row gid,   token 2*tig
      split_tf32(s[nb][2], ah[1], al[1]);   // row gid+8, token 2*tig
      split_tf32(s[nb][1], ah[2], al[2]);   // row gid,   token 2*tig+1
      split_tf32(s[nb][3], ah[3], al[3]);   // row gid+8, token 2*tig+1
      const float* vp = vt + (nb * 8 + 2 * tig) * QS + gid;
#pragma unroll
      for (int ob0 = 0; ob0 < KS; ob0 += 4) {
        uint32_t h0[4], g0[4], h1[4], g1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          split_tf32(vp[(ob0 + i) * 8], h0[i], g0[i]);
          split_tf32(vp[QS + (ob0 + i) * 8], h1[i], g1[i]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_tf32(o[ob0 + i], al, h0[i], h1[i]);
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_tf32(o[ob0 + i], ah, g0[i], g1[i]);
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_tf32(o[ob0 + i], ah, h0[i], h1[i]);
      }
    }
    __syncthreads();   // the next iteration's copies overwrite the other stage only after everyone left it
  }

  // ---- normalise and store --------------------------------------------------------------------------------------
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = 1.0f / fmaxf(l0, 1e-12f), inv1 = 1.0f / fmaxf(l1, 1e-12f);
  if (en0 < p.B) {
    float* dst = p.out + (size_t)en0 * p.out_stride + (size_t)(kvh * G + r0 % G) * HD + 2 * tig;
#pragma unroll
    for (int ob = 0; ob < KS; ++ob) *reinterpret_cast<float2*>(dst + ob * 8) = make_float2(o[ob][0] * inv0, o[ob][1] * inv0);
  }
  if (en1 < p.B) {
    float* dst = p.out + (size_t)en1 * p.out_stride + (size_t)(kvh * G + r1 % G) * HD + 2 * tig;
#pragma unroll
    for (int ob = 0; ob < KS; ++ob) *reinterpret_cast<float2*>(dst + ob * 8) = make_float2(o[ob][2] * inv1, o[ob][3] * inv1);
  }
}

template <int HD, int G>
cudaError_t launch_one(pi_ctx* ctx, dim3 grid, const SharedAttnParams& p) {
  auto k = attn_shared_table_kernel<HD, G>;
  constexpr size_t smem = (size_t)(2 * kRows + 4 * kTile) * (HD + 4) * sizeof(float);
  static pi_smem_grant granted;
  if (smem > granted.of(ctx)) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    granted.of(ctx) = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, k, p);
}

template <int HD>
cudaError_t launch_group(pi_ctx* ctx, int group, dim3 grid, const SharedAttnParams& p) {
  switch (group) {
    case 1: return launch_one<HD, 1>(ctx, grid, p);
    case 2: return launch_one<HD, 2>(ctx, grid, p);
    case 4: return launch_one<HD, 4>(ctx, grid, p);
    default: return launch_one<HD, 8>(ctx, grid, p);
  }
}

}  // namespace

// Whether the shared-table kernel takes this batch: every entry maps the same table, the geometry is one the kernel
// is built for, and there are enough row tiles to fill the GPU (the kernel does not split the KV axis, so a short
// chunk is better served by the decode kernel's KV splits).  opt_attn_shared: 0 never, 1 by this rule, 2 whenever
// the geometry allows.
bool pi_attention_shared_usable(const pi_ctx* ctx, const pi_kv_pool* pool, int num_heads, const float* q, size_t q_stride,
                                const float* out, size_t out_stride, const pi_attn_batch& batch) {
  if (!ctx->opt_attn_shared || !batch.shared_table || batch.B < 2) return false;
  const pi_kv_layout& L = pool->L;
  const int HD = L.head_dim, group = num_heads / L.num_kv_heads;
  if (!(HD == 64 || HD == 128) || !(group == 1 || group == 2 || group == 4 || group == 8) || L.block_size != kBlock) return false;
  if ((uintptr_t)q % 16 || q_stride % 4 || (uintptr_t)out % 8 || out_stride % 2) return false;
  const size_t smem = (size_t)(2 * kRows + 4 * kTile) * (HD + 4) * sizeof(float);
  if (smem + 1024 > ctx->smem_optin) return false;
  if (ctx->opt_attn_shared >= 2) return true;
  if (pi_attention_shared_tc_usable(ctx, pool, num_heads, q, q_stride, out, out_stride)) {
    // tcgen05 kernel: 128 rows per CTA; worth it from about a quarter of the SMs on
    const long ctas_tc = (long)L.num_kv_heads * (((long)batch.B * group + 127) / 128);
    return ctas_tc * 4 >= ctx->sm_count;
  }
  const long ctas = (long)L.num_kv_heads * ((batch.B + kRows / group - 1) / (kRows / group));
  return ctas * 4 >= (long)ctx->sm_count * 3;   // measured: break-even near 3/4 of the SMs, 1.3-2x faster from one CTA per SM on
}

pi_status pi_launch_attention_shared(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q,
                                     size_t q_stride, float* out, size_t out_stride, const pi_attn_batch& batch) {
  const pi_kv_layout& L = pool->L;
  const int HD = L.head_dim, group = num_heads / L.num_kv_heads;
  // head_dim 64: the tcgen05 kernel (opt_attn_shared 3 keeps this mma.sync kernel, for comparison)
  if (ctx->opt_attn_shared != 3 && pi_attention_shared_tc_usable(ctx, pool, num_heads, q, q_stride, out, out_stride))
    return pi_launch_attention_shared_tc(ctx, pool, layer, num_heads, q, q_stride, out, out_stride, batch);
  SharedAttnParams p;
  p.q = q;
  p.q_stride = q_stride;
  p.out = out;
  p.out_stride = out_stride;
  p.kv = pool->data;
  p.L = L;
  p.layer = layer;
  p.B = batch.B;
  p.table = batch.tables;   // row 0 = every row
  p.len = batch.shared_len;
  p.pos = batch.pos;
  p.start = batch.start;
  p.scale2 = (1.0f / sqrtf((float)HD)) * 1.4426950408889634f;
  const int ppc = kRows / group;
  const dim3 grid(L.num_kv_heads, (batch.B + ppc - 1) / ppc);
  const cudaError_t e = HD == 64 ? launch_group<64>(ctx, group, grid, p) : launch_group<128>(ctx, group, grid, p);
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "shared-table attention launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  return PI_OK;
}
