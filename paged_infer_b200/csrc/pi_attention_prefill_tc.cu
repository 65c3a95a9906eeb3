// Shared-table paged attention on the 5th-generation tensor cores (tcgen05, accumulators and the A operands in
// tensor memory), head_dim 64.  Same contract as the mma.sync kernel in pi_attention_prefill.cu: the entries of the
// batch map ONE block table (the positions of a prefill chunk, a speculative verify group; reference
// src/model.rs:1222-1255, src/attention.rs:141-265); entry e attends start[e]..=pos[e]; unmapped blocks score -inf
// and are never read; an empty window gives zeros.
//
// One CTA owns 128 query rows - (position, query head) pairs of one KV head, one row per TMEM lane - and walks the
// window in tiles of 64 tokens.  Every f32 value x is carried as three bf16 planes x0 + x1 + x2 = x (exact), and a
// product of two split values keeps the six terms down to 2^-24:  a0 b0 + (a0 b1 + a1 b0) + (a0 b2 + a1 b1 + a2 b0).
// These are six MMAs (M = 128, N = 64, K = 16) per K step, one per plane pair (i, j) with i + j <= 2, smallest terms
// first, all into the SAME 64 accumulator columns: every product of two bf16 is exact in the f32 accumulator, so the
// columns hold an f32 dot product of the terms and the softmax threads read 64 columns per tile.
//
//   scores  S = Q K^T : A = the planes of Q (tensor memory, written once), B = the planes of the K tile
//                       (shared memory, K-major, 128-byte swizzle, rows = tokens)
//   output  O = P V   : A = the planes of P (tensor memory, written by the softmax threads, two buffers),
//                       B = the planes of V^T (rows = head dims, K = tokens); the product of one tile lands in scratch
//                       columns and is folded into the running output with the online-softmax correction
//
// Warp roles: 0-3 = one thread per query row (read S, mask, online softmax in the log2 domain, write P, read the
// tile's O and fold it into the running f32 output held in registers); 4-7 = converters (request the next K/V tile
// from the pool, split the current one into planes, store swizzled: K as is, V transposed; up to four tiles ahead
// of the MMAs); 8 = TMEM allocation and the MMA issuer (the scores of tile j+1 are issued before the output product
// of tile j, so they run while the row threads work on tile j).  Hand-offs go through mbarriers; every wait is
// bounded and raises the context's error word instead of hanging.  Measured and dropped: two threads per row with
// the row maximum exchanged through shared memory (the extra hand-off per tile cost more than the halved work).
#include <math.h>

#include <algorithm>

#include "pi_common.cuh"

namespace {

constexpr int kHD = 64;
constexpr int kRowsTc = 128;       // query rows per CTA = TMEM lanes
constexpr int kTileTc = 64;        // tokens per tile
constexpr int kBlockTc = 16;
constexpr int kThreadsTc = 9 * 32;
constexpr uint32_t kSpinTc = 1u << 21;
constexpr int kPlaneTileBytes = 3 * 64 * 128;          // three planes x 64 rows x 128 bytes
constexpr int kStageBytesTc = 2 * kPlaneTileBytes;     // K planes + V^T planes
constexpr int kStagesTc = 4;                           // K/V plane tiles in flight
constexpr size_t kSmemTc = (size_t)kStagesTc * kStageBytesTc + 1024;
// TMEM columns: two score buffers, two buffers of P planes (3 x 32 columns each), the tile's output, the Q planes
constexpr uint32_t kColS = 0, kColP = 128, kColO = 320, kColQ = 384;

struct TcAttnParams {
  const float* q;
  size_t q_stride;
  float* out;
  size_t out_stride;
  const float* kv;
  pi_kv_layout L;
  int layer;
  int B;
  int group;              // query heads per KV head
  const int32_t* table;
  int len;
  const int32_t* pos;
  const int32_t* start;
  float scale2;
  int* err_flag;
};

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kSpinTc; ++spin) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ float ex2a(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void t_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void t_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// 64 consecutive columns of this thread's lane.
__device__ __forceinline__ void t_ld64(uint32_t base, float* v) {
  uint32_t r[64];
#pragma unroll
  for (int c = 0; c < 4; ++c) t_ld16(base + (uint32_t)(c * 16), r + c * 16);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// The three planes of a pair of values, packed (x in the low half): same roundings as pi_split3, two values per
// conversion instruction.
__device__ __forceinline__ void split3_pair(float x, float y, uint32_t& w0, uint32_t& w1, uint32_t& w2) {
  __nv_bfloat162 a = __floats2bfloat162_rn(x, y);
  w0 = *reinterpret_cast<uint32_t*>(&a);
  const float rx = x - __uint_as_float(w0 << 16), ry = y - __uint_as_float(w0 & 0xffff0000u);
  __nv_bfloat162 b = __floats2bfloat162_rn(rx, ry);
  w1 = *reinterpret_cast<uint32_t*>(&b);
  const float sx = rx - __uint_as_float(w1 << 16), sy = ry - __uint_as_float(w1 & 0xffff0000u);
  __nv_bfloat162 c = __floats2bfloat162_rn(sx, sy);
  w2 = *reinterpret_cast<uint32_t*>(&c);
}
// The planes of 16 values as packed bf16 pairs (value 2i in the low half of word i).
__device__ __forceinline__ void planes16(const float* x, uint32_t* w0, uint32_t* w1, uint32_t* w2) {
#pragma unroll
  for (int i = 0; i < 8; ++i) split3_pair(x[2 * i], x[2 * i + 1], w0[i], w1[i], w2[i]);
}

// Lane 0 polls for the warp.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int lane) {
  int ok = 1;
  if (lane == 0) ok = (!*abort_flag && bar_wait(bar, parity)) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__global__ void __launch_bounds__(kThreadsTc, 1) attn_shared_tc_kernel(const TcAttnParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw_tc[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw_tc + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bars[2 * kStagesTc + 6];
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_abort;
  __shared__ int s_lo, s_hi;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.group, ppc = kRowsTc / G;
  const int kvh = blockIdx.x;
  const int e0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * ppc;   // long windows first
  // per stage / buffer: kv_full, kv_free, s_full, p_full (index parity of the tile); single: o_full, o_free
  const uint32_t kv_full0 = s_u32(&bars[0]), kv_free0 = s_u32(&bars[kStagesTc]), s_full0 = s_u32(&bars[2 * kStagesTc]),
                 p_full0 = s_u32(&bars[2 * kStagesTc + 2]), o_full = s_u32(&bars[2 * kStagesTc + 4]),
                 o_free = s_u32(&bars[2 * kStagesTc + 5]);
  if (tid == 0) {
    for (int i = 0; i < kStagesTc; ++i) {
      bar_init(kv_full0 + 8 * i, 4);   // one arrival per converter warp
      bar_init(kv_free0 + 8 * i, 1);   // tcgen05.commit
    }
    for (int i = 0; i < 2; ++i) {
      bar_init(s_full0 + 8 * i, 1);    // tcgen05.commit
      bar_init(p_full0 + 8 * i, 4);    // one arrival per row warp
    }
    bar_init(o_full, 1);
    bar_init(o_free, 4);
    s_abort = 0;
    s_lo = 0x7fffffff;
    s_hi = -1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(&s_tmem)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // the dependent grid is released only now that this CTA holds its tensor memory (a dependent CTA that took the
  // SM's columns first would keep them until this grid completes)
  pi_grid_launch_dependents();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;
  const uint32_t smem_base = s_u32(smem);
  pi_grid_dependency_wait();

  if (tid < ppc && e0 + tid < p.B) {
    const int ps = p.pos[e0 + tid], st = p.start[e0 + tid];
    if (st <= ps) {
      atomicMin(&s_lo, st);
      atomicMax(&s_hi, ps);
    }
  }
  // the row of this thread (warps 0-3) and its Q planes
  const int en = e0 + tid / G, hq = kvh * G + tid % G;
  const bool row_valid = warp < 4 && en < p.B;
  const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  int pos_r = -1, st_r = 0;
  if (warp < 4) {
    if (row_valid) {
      pos_r = p.pos[en];
      st_r = p.start[en];
    }
    const float* qrow = p.q + (size_t)(row_valid ? en : 0) * p.q_stride + (size_t)hq * kHD;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float x[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row_valid) v = __ldg(reinterpret_cast<const float4*>(qrow + half * 32 + i * 4));
        x[4 * i] = v.x * p.scale2;
        x[4 * i + 1] = v.y * p.scale2;
        x[4 * i + 2] = v.z * p.scale2;
        x[4 * i + 3] = v.w * p.scale2;
      }
      uint32_t w0[16], w1[16], w2[16];
      planes16(x, w0, w1, w2);
      planes16(x + 16, w0 + 8, w1 + 8, w2 + 8);
      t_st16(lane_addr + kColQ + 0 * 32 + half * 16, w0);
      t_st16(lane_addr + kColQ + 1 * 32 + half * 16, w1);
      t_st16(lane_addr + kColQ + 2 * 32 + half * 16, w2);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const int t_min = s_lo, t_max = s_hi;
  const int jt_first = t_max >= 0 ? t_min / kTileTc : 0;
  const int ntiles = t_max >= 0 ? t_max / kTileTc - jt_first + 1 : 0;
  auto block_of = [&](int lb) -> int {
    if (lb >= p.len || lb * kBlockTc > t_max || lb * kBlockTc + kBlockTc - 1 < t_min) return -1;
    return p.table[lb];
  };
  auto fail = [&](int code) {
    if (!s_abort) {
      s_abort = 1;
      if (p.err_flag) atomicExch(p.err_flag, code);
    }
  };

  float acc[kHD];
#pragma unroll
  for (int i = 0; i < kHD; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  if (warp < 4) {
    // ---- one thread per query row ------------------------------------------------------------------------------
    float corr_prev = 1.f;
    bool alive = true;
    // the output of tile j (P relative to the running maximum after tile j) folded into the running output
    auto fold_output = [&](int j, float corr) -> bool {
      if (!warp_wait(o_full, j & 1, &s_abort, lane)) {
        if (lane == 0) fail(12);
        return false;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t o[32];
        t_ld16(lane_addr + kColO + h * 32, o);
        t_ld16(lane_addr + kColO + h * 32 + 16, o + 16);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[h * 32 + i] = acc[h * 32 + i] * corr + __uint_as_float(o[i]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive(o_free);
      return true;
    };
    for (int j = 0; j < ntiles; ++j) {
      const int jt = jt_first + j, buf = j & 1;
      if (!warp_wait(s_full0 + 8 * buf, (j >> 1) & 1, &s_abort, lane)) {
        if (lane == 0) fail(11);
        alive = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float s[kTileTc];
      t_ld64(lane_addr + kColS + buf * 64, s);
      unsigned mapped = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) mapped |= (block_of(jt * 4 + i) >= 0 ? 1u : 0u) << i;
      // a tile that lies wholly inside the window of every row of the warp needs no masks
      const bool inside = mapped == 0xFu && jt * kTileTc >= st_r && jt * kTileTc + kTileTc - 1 <= pos_r;
      if (!__all_sync(0xffffffffu, inside)) {
#pragma unroll
        for (int i = 0; i < kTileTc; ++i) {
          const int t = jt * kTileTc + i;
          const bool ok = ((mapped >> (i >> 4)) & 1u) && t >= st_r && t <= pos_r;
          s[i] = ok ? s[i] : -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one of 64 links
#pragma unroll
      for (int i = 0; i < kTileTc; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], s[i]);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_run, mx);
      const float corr = (m_run == -INFINITY) ? 1.f : ex2a(m_run - m_new);
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < kTileTc; ++i) {
        s[i] = (s[i] == -INFINITY) ? 0.f : ex2a(s[i] - m_new);
        ps4[i & 3] += s[i];
      }
      const float psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      l_run = l_run * corr + psum;
      m_run = m_new;
      // the previous tile's output is ready by now (its MMAs were issued when its P was handed over): fold it in and
      // free the output columns for this tile's product
      if (j > 0 && !fold_output(j - 1, corr_prev)) {
        alive = false;
        break;
      }
      corr_prev = corr;
      // P planes of this tile: plane pl at column pl * 32 of the buffer, two tokens per column
      const uint32_t pcol = lane_addr + kColP + buf * 96;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t w0[16], w1[16], w2[16];
        planes16(s + half * 32, w0, w1, w2);
        planes16(s + half * 32 + 16, w0 + 8, w1 + 8, w2 + 8);
        t_st16(pcol + 0 * 32 + half * 16, w0);
        t_st16(pcol + 1 * 32 + half * 16, w1);
        t_st16(pcol + 2 * 32 + half * 16, w2);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive(p_full0 + 8 * buf);
    }
    if (alive && ntiles > 0) fold_output(ntiles - 1, corr_prev);
    if (row_valid) {
      const float inv = 1.0f / fmaxf(l_run, 1e-12f);
      float* dst = p.out + (size_t)en * p.out_stride + (size_t)hq * kHD;
#pragma unroll
      for (int i = 0; i < kHD / 4; ++i)
        *reinterpret_cast<float4*>(dst + 4 * i) = make_float4(acc[4 * i] * inv, acc[4 * i + 1] * inv, acc[4 * i + 2] * inv, acc[4 * i + 3] * inv);
    }
  } else if (warp < 8) {
    // ---- converters: planes of the K tile (rows = tokens) and of the V tile transposed (rows = head dims) ---------
    // Thread ct: K items (token ct/8 + 16*it, dims 8*(ct%8)..+7) and V items (head dim ct%64, tokens 8g..8g+7 with
    // g = ct/64 + 2*it), it = 0..3: item `it` of either kind lies in block `it` of the tile.  The values of the NEXT
    // tile are requested before the current ones are converted, so the pool's latency is off the path.
    const int ct = tid - 128;
    const int ktok = ct >> 3, kc = ct & 7, vd_ = ct & 63, vg = ct >> 6;
    float cur[64], nxt[64];
    auto fetch = [&](int jt, float* r) {
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int b = block_of(jt * 4 + it);
        const int tok = ktok + 16 * it, t = jt * kTileTc + tok;
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f), v = u;
        if (b >= 0 && t >= t_min && t <= t_max) {
          const float* src = p.kv + pi_kv_tile_offset(p.L, p.layer, b, kvh, 0) + ktok * kHD + kc * 8;
          u = __ldg(reinterpret_cast<const float4*>(src));
          v = __ldg(reinterpret_cast<const float4*>(src + 4));
        }
        r[it * 8 + 0] = u.x; r[it * 8 + 1] = u.y; r[it * 8 + 2] = u.z; r[it * 8 + 3] = u.w;
        r[it * 8 + 4] = v.x; r[it * 8 + 5] = v.y; r[it * 8 + 6] = v.z; r[it * 8 + 7] = v.w;
        const float* vsrc = p.kv + pi_kv_tile_offset(p.L, p.layer, b >= 0 ? b : 0, kvh, 1) + vd_;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int tk = (vg + 2 * it) * 8 + e, tt = jt * kTileTc + tk;   // tk / 16 == it
          r[32 + it * 8 + e] = (b >= 0 && tt >= t_min && tt <= t_max) ? __ldg(vsrc + (tk & 15) * kHD) : 0.f;
        }
      }
    };
    if (ntiles > 0) fetch(jt_first, cur);
    for (int j = 0; j < ntiles; ++j) {
      const int stg = j % kStagesTc;
      if (j + 1 < ntiles) fetch(jt_first + j + 1, nxt);
      if (!warp_wait(kv_free0 + 8 * stg, ((j / kStagesTc) & 1) ^ 1, &s_abort, lane)) {
        if (lane == 0) fail(13);
        break;
      }
      unsigned char* kdst = smem + (size_t)stg * kStageBytesTc;
      unsigned char* vdst = kdst + kPlaneTileBytes;
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        uint32_t w0[4], w1[4], w2[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) split3_pair(cur[it * 8 + 2 * i], cur[it * 8 + 2 * i + 1], w0[i], w1[i], w2[i]);
        const int tok = ktok + 16 * it;
        const int off = tok * 128 + ((kc ^ (tok & 7)) << 4);
        *reinterpret_cast<uint4*>(kdst + 0 * 8192 + off) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
        *reinterpret_cast<uint4*>(kdst + 1 * 8192 + off) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
        *reinterpret_cast<uint4*>(kdst + 2 * 8192 + off) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
      }
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        uint32_t w0[4], w1[4], w2[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) split3_pair(cur[32 + it * 8 + 2 * i], cur[32 + it * 8 + 2 * i + 1], w0[i], w1[i], w2[i]);
        const int g = vg + 2 * it;
        const int off = vd_ * 128 + ((g ^ (vd_ & 7)) << 4);
        *reinterpret_cast<uint4*>(vdst + 0 * 8192 + off) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
        *reinterpret_cast<uint4*>(vdst + 1 * 8192 + off) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
        *reinterpret_cast<uint4*>(vdst + 2 * 8192 + off) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA's reads
      __syncwarp();
      if (lane == 0) bar_arrive(kv_full0 + 8 * stg);
#pragma unroll
      for (int i = 0; i < 64; ++i) cur[i] = nxt[i];
    }
  } else if (lane == 0) {
    // ---- MMA issuer ------------------------------------------------------------------------------------------------
    auto idesc = [](uint32_t n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(kRowsTc >> 4) << 24); };
    const uint32_t id64 = idesc(64);
    // D[128 x 64] (+)= sum over the six plane pairs (i, j), i + j <= 2, of A plane i (TMEM) x B plane j (shared), for
    // the four K steps of a tile: everything lands in the same 64 accumulator columns, smallest terms first.
    auto product = [&](uint32_t d_col, uint32_t a_col, uint32_t b_addr) {
      const uint64_t bd = desc_sw128(b_addr);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {   // 16 K elements: 8 TMEM columns of an A plane, 32 bytes of every B row
        const int pi[6] = {0, 1, 2, 0, 1, 0}, pj[6] = {2, 1, 0, 1, 0, 0};
#pragma unroll
        for (int t = 0; t < 6; ++t)
          mma_ts(tmem + d_col, tmem + a_col + pi[t] * 32 + ks * 8, bd + (uint64_t)((pj[t] * 8192 + ks * 32) >> 4), id64,
                 (ks > 0 || t > 0) ? 1u : 0u);
      }
    };
    auto scores = [&](int j) -> bool {
      const int stg = j % kStagesTc, buf = j & 1;
      if (s_abort || !bar_wait(kv_full0 + 8 * stg, (j / kStagesTc) & 1)) {
        fail(14);
        return false;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      product(kColS + buf * 64, kColQ, smem_base + stg * kStageBytesTc);
      mma_commit(s_full0 + 8 * buf);
      return true;
    };
    bool ok = ntiles > 0 && scores(0);
    for (int j = 0; j < ntiles && ok; ++j) {
      const int stg = j % kStagesTc, buf = j & 1;
      // the next tile's scores run on the tensor pipe while the row threads work on this tile's softmax
      if (j + 1 < ntiles && !scores(j + 1)) break;
      if (s_abort || !bar_wait(p_full0 + 8 * buf, (j >> 1) & 1) || (j > 0 && !bar_wait(o_free, (j - 1) & 1))) {
        fail(15);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      product(kColO, kColP + buf * 96, smem_base + stg * kStageBytesTc + kPlaneTileBytes);
      mma_commit(o_full);
      mma_commit(kv_free0 + 8 * stg);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 8) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
  }
}

}  // namespace

bool pi_attention_shared_tc_usable(const pi_ctx* ctx, const pi_kv_pool* pool, int num_heads, const float* q, size_t q_stride,
                                   const float* out, size_t out_stride) {
  const pi_kv_layout& L = pool->L;
  const int group = num_heads / L.num_kv_heads;
  return L.head_dim == kHD && L.block_size == kBlockTc && (group == 1 || group == 2 || group == 4 || group == 8) &&
         (uintptr_t)q % 16 == 0 && q_stride % 4 == 0 && (uintptr_t)out % 16 == 0 && out_stride % 4 == 0 &&
         std::max(kSmemTc, (size_t)120 * 1024) + 1024 <= ctx->smem_optin;
}

pi_status pi_launch_attention_shared_tc(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q,
                                        size_t q_stride, float* out, size_t out_stride, const pi_attn_batch& batch) {
  const pi_kv_layout& L = pool->L;
  TcAttnParams p;
  p.q = q;
  p.q_stride = q_stride;
  p.out = out;
  p.out_stride = out_stride;
  p.kv = pool->data;
  p.L = L;
  p.layer = layer;
  p.B = batch.B;
  p.group = num_heads / L.num_kv_heads;
  p.table = batch.tables;
  p.len = batch.shared_len;
  p.pos = batch.pos;
  p.start = batch.start;
  p.scale2 = (1.0f / sqrtf((float)kHD)) * 1.4426950408889634f;
  p.err_flag = ctx->dev_err;
  // At least 120 KB of shared memory per CTA: two of these CTAs (each wants all 512 TMEM columns) never share an SM.
  const size_t smem = std::max(kSmemTc, (size_t)120 * 1024);
  static pi_smem_grant granted;
  if (smem > granted.of(ctx)) {
    const cudaError_t e = cudaFuncSetAttribute(attn_shared_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "shared-table attention: %s", cudaGetErrorString(e));
    granted.of(ctx) = smem;
  }
  const int ppc = kRowsTc / p.group;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(L.num_kv_heads, (batch.B + ppc - 1) / ppc);
  cfg.blockDim = dim3(kThreadsTc);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, attn_shared_tc_kernel, p);
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "shared-table attention launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  return PI_OK;
}
