// Paged-attention decode over the device-resident KV pool.
//
// Entry b (one query position of one sequence) attends positions
// start[b]..=pos[b]; logical block t / block_size is looked up once per block in
// the entry's block-table row; a logical block past the mapped length scores
// -inf (it is skipped: its K and V are never touched); an empty or fully masked
// window gives zeros.  Query head h reads KV head h / kv_group.
//
// Fast path (head_dim 64 or 128, kv_group 1/2/4/8): one CTA per (kv head, entry,
// KV split).  Each warp walks whole physical blocks; head_dim/8 lanes share a
// token, each lane holding 8 dims of every query head of the group, so one
// 2 x 128-bit load of K and of V per lane serves all kv_group query heads.
// Softmax is online (running max / sum per head); warps and KV splits are merged
// by log-sum-exp.  Generic path (any head_dim <= 512, any group, any block
// size): one warp per (entry, query head).
//
// Replaces PagedAttention::run and for_each_block (reference
// src/attention.rs:141-295), math::softmax_in_place (src/math.rs:405-426) and
// BlockTable::get_physical_location (src/memory/block_table.rs:50-61).
#include <math.h>

#include <string.h>

#include <algorithm>

#include "pi_common.cuh"
#include "pi_attention.cuh"

namespace {

constexpr int kAttnWarps = 4;

struct AttnParams {
  const float* q;
  size_t q_stride;
  float* out;
  size_t out_stride;
  const float* kv;
  pi_kv_layout L;
  int layer;
  int H;
  const int32_t* tables;
  int max_blocks;
  const int32_t* lens;
  const int32_t* pos;
  const int32_t* start;
  const int32_t* safe_lb;   // [B] or null: blocks below this index may be fetched before the dependency wait
  int blocks_per_cta;
  int nsplit;
  float* part_ml;   // [B][H][nsplit][2]
  float* part_acc;  // [B][H][nsplit][HD]
  float scale;
  int* err_flag;
  unsigned short* emit_base;   // merge kernel only: out as three bf16 planes [3][.][emit_k], or null
  size_t emit_plane_stride;
  int emit_k;
};

__device__ __forceinline__ float4 ldg_f4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

// Merge (m, l, acc...) pairs: factor for a side with running max `m` once the joint max is `M`.
__device__ __forceinline__ float lse_factor(float m, float M) { return m == -INFINITY ? 0.f : __expf(m - M); }

template <int HD, int G>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode_kernel(const AttnParams p) {
  constexpr int LPT = HD / 8;    // lanes per token
  constexpr int TPW = 32 / LPT;  // tokens per warp step
  __shared__ float s_acc[kAttnWarps][G][HD];
  __shared__ float s_m[kAttnWarps][G], s_l[kAttnWarps][G];

  pi_grid_dependency_wait();
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tg = lane / LPT, li = lane % LPT;
  const int BS = p.L.block_size;
  const int pos = p.pos[b], st = p.start[b], len = p.lens[b];
  const int lb_first = st / BS, lb_last = pos / BS;
  const int lb_begin = lb_first + split * p.blocks_per_cta;
  const int lb_end = min(min(lb_last + 1, lb_begin + p.blocks_per_cta), len);  // unmapped tail is masked

  float qv[G][8];
  const float* qb = p.q + (size_t)b * p.q_stride + (size_t)kvh * G * HD + li * 8;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float4 a = ldg_f4(qb + g * HD), c = ldg_f4(qb + g * HD + 4);
    qv[g][0] = a.x; qv[g][1] = a.y; qv[g][2] = a.z; qv[g][3] = a.w;
    qv[g][4] = c.x; qv[g][5] = c.y; qv[g][6] = c.z; qv[g][7] = c.w;
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }

  if (st <= pos) {
    for (int lb = lb_begin + warp; lb < lb_end; lb += kAttnWarps) {
      const int pb = p.tables[(size_t)b * p.max_blocks + lb];
      const int t_lo = max(st - lb * BS, 0), t_hi = min(pos - lb * BS, BS - 1);
      const float* Kt = p.kv + pi_kv_tile_offset(p.L, p.layer, pb, kvh, 0) + li * 8;
      const float* Vt = Kt + (size_t)BS * HD;
      for (int t0 = t_lo; t0 <= t_hi; t0 += TPW) {
        const int t = t0 + tg;
        const bool valid = t <= t_hi;
        float kx[8], vx[8];
        if (valid) {
          const float4 k0 = ldg_f4(Kt + (size_t)t * HD), k1 = ldg_f4(Kt + (size_t)t * HD + 4);
          const float4 v0 = ldg_f4(Vt + (size_t)t * HD), v1 = ldg_f4(Vt + (size_t)t * HD + 4);
          kx[0] = k0.x; kx[1] = k0.y; kx[2] = k0.z; kx[3] = k0.w; kx[4] = k1.x; kx[5] = k1.y; kx[6] = k1.z; kx[7] = k1.w;
          vx[0] = v0.x; vx[1] = v0.y; vx[2] = v0.z; vx[3] = v0.w; vx[4] = v1.x; vx[5] = v1.y; vx[6] = v1.z; vx[7] = v1.w;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) kx[i] = vx[i] = 0.f;
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float d = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) d = fmaf(qv[g][i], kx[i], d);
#pragma unroll
          for (int o = 1; o < LPT; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          const float s = valid ? d * p.scale : -INFINITY;
          if (s > m[g]) {  // uniform across the LPT lanes of a token
            const float corr = lse_factor(m[g], s);
            l[g] *= corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[g][i] *= corr;
            m[g] = s;
          }
          const float w = valid ? __expf(s - m[g]) : 0.f;
          l[g] += w;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(w, vx[i], acc[g][i]);
        }
      }
    }
  }

  // merge the token groups of the warp
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o), lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float M = fmaxf(m[g], mo);
      const float fs = lse_factor(m[g], M), fo = lse_factor(mo, M);
      l[g] = l[g] * fs + lo * fo;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][i], o);
        acc[g][i] = acc[g][i] * fs + ao * fo;
      }
      m[g] = M;
    }
  }
  if (tg == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int i = 0; i < 8; ++i) s_acc[warp][g][li * 8 + i] = acc[g][i];
      if (li == 0) {
        s_m[warp][g] = m[g];
        s_l[warp][g] = l[g];
      }
    }
  }
  __syncthreads();
  pi_grid_launch_dependents();

  // merge the warps; write the result or this split's partial
  for (int idx = tid; idx < G * HD; idx += kAttnWarps * 32) {
    const int g = idx / HD, d = idx - g * HD;
    float M = s_m[0][g];
#pragma unroll
    for (int w = 1; w < kAttnWarps; ++w) M = fmaxf(M, s_m[w][g]);
    float ls = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float f = lse_factor(s_m[w][g], M);
      ls += s_l[w][g] * f;
      a += s_acc[w][g][d] * f;
    }
    const int h = kvh * G + g;
    if (p.nsplit == 1) {
      p.out[(size_t)b * p.out_stride + (size_t)h * HD + d] = a * (1.0f / fmaxf(ls, 1e-12f));
    } else {
      const size_t slot = ((size_t)b * p.H + h) * p.nsplit + split;
      p.part_acc[slot * HD + d] = a;
      if (d == 0) {
        p.part_ml[slot * 2] = M;
        p.part_ml[slot * 2 + 1] = ls;
      }
    }
  }
}

// Same work split as attn_decode_kernel, but every (block, kv head) K|V tile - one contiguous
// 2*block_size*HD*4-byte span of the pool - is brought into shared memory by a bulk async copy
// (TMA, cp.async.bulk) through a per-warp ring of STAGES slots, so several tiles per warp are in
// flight while one is being consumed.  A lane reads 16-byte chunks `li` and `li + LPT` of a token
// row, which keeps the 128-bit shared loads free of bank conflicts.
template <int HD, int G, int STAGES>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode_tma_kernel(const AttnParams p) {
  constexpr int LPT = HD / 8;    // lanes per token
  constexpr int TPW = 32 / LPT;  // tokens per warp step
  extern __shared__ __align__(128) unsigned char attn_smem[];
  __shared__ __align__(8) unsigned long long bars[kAttnWarps][STAGES];
  __shared__ float s_m[kAttnWarps][G], s_l[kAttnWarps][G];

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tg = lane / LPT, li = lane % LPT;
  const int BS = p.L.block_size;
  const uint32_t tile_bytes = 2u * BS * HD * sizeof(float);
  float* ring = reinterpret_cast<float*>(attn_smem) + (size_t)warp * STAGES * (tile_bytes / 4);

  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(attn_smem_u32(&bars[warp][s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  pi_grid_dependency_wait();

  const int pos = p.pos[b], st = p.start[b], len = p.lens[b];
  const int lb_first = st / BS, lb_last = pos / BS;
  const int lb_begin = lb_first + split * p.blocks_per_cta;
  const int lb_end = min(min(lb_last + 1, lb_begin + p.blocks_per_cta), len);
  const int nblk = (st <= pos && lb_begin + warp < lb_end) ? (lb_end - lb_begin - warp + kAttnWarps - 1) / kAttnWarps : 0;

  auto issue = [&](int j) {  // lane 0 only: tile j of this warp -> slot j % STAGES
    const int lb = lb_begin + warp + j * kAttnWarps;
    const int pb = p.tables[(size_t)b * p.max_blocks + lb];
    const float* src = p.kv + pi_kv_tile_offset(p.L, p.layer, pb, kvh, 0);
    const uint32_t bar = attn_smem_u32(&bars[warp][j % STAGES]);
    const uint32_t dst = attn_smem_u32(ring + (size_t)(j % STAGES) * (tile_bytes / 4));
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tile_bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(tile_bytes), "r"(bar)
                 : "memory");
  };
  if (lane == 0)
    for (int j = 0; j < STAGES && j < nblk; ++j) issue(j);

  float qv[G][8];
  const float* qb = p.q + (size_t)b * p.q_stride + (size_t)kvh * G * HD;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float4 a = ldg_f4(qb + g * HD + li * 4), c = ldg_f4(qb + g * HD + (li + LPT) * 4);
    qv[g][0] = a.x; qv[g][1] = a.y; qv[g][2] = a.z; qv[g][3] = a.w;
    qv[g][4] = c.x; qv[g][5] = c.y; qv[g][6] = c.z; qv[g][7] = c.w;
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }

  bool failed = false;
  for (int j = 0; j < nblk && !failed; ++j) {
    const int slot = j % STAGES;
    const uint32_t bar = attn_smem_u32(&bars[warp][slot]);
    const uint32_t parity = (j / STAGES) & 1;
    uint32_t done = 0;
    for (uint32_t spin = 0; spin < kAttnSpinLimit && !done; ++spin)
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (!__all_sync(0xffffffffu, done != 0)) {  // the copy never landed: report and stop (the result is not trusted)
      if (lane == 0 && p.err_flag) atomicExch(p.err_flag, 6);
      failed = true;
      // give the copies still in flight one more bounded chance to land before the CTA's memory is released
      for (int jj = j + 1; jj < nblk && jj < j + STAGES; ++jj) {
        const uint32_t b2 = attn_smem_u32(&bars[warp][jj % STAGES]), par2 = (jj / STAGES) & 1;
        uint32_t d2 = 0;
        for (uint32_t spin = 0; spin < kAttnSpinLimit && !d2; ++spin)
          asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                       : "=r"(d2) : "r"(b2), "r"(par2) : "memory");
      }
      break;
    }
    const int lb = lb_begin + warp + j * kAttnWarps;
    const int t_lo = max(st - lb * BS, 0), t_hi = min(pos - lb * BS, BS - 1);
    const float* Kt = ring + (size_t)slot * (tile_bytes / 4);
    const float* Vt = Kt + (size_t)BS * HD;
    for (int t0 = t_lo; t0 <= t_hi; t0 += TPW) {
      const int t = t0 + tg;
      const bool valid = t <= t_hi;
      const int tc = valid ? t : t_hi;  // clamp: the row is in shared memory either way
      const float4 k0 = *reinterpret_cast<const float4*>(Kt + (size_t)tc * HD + li * 4);
      const float4 k1 = *reinterpret_cast<const float4*>(Kt + (size_t)tc * HD + (li + LPT) * 4);
      const float4 v0 = *reinterpret_cast<const float4*>(Vt + (size_t)tc * HD + li * 4);
      const float4 v1 = *reinterpret_cast<const float4*>(Vt + (size_t)tc * HD + (li + LPT) * 4);
      const float kx[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
      const float vx[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d = fmaf(qv[g][i], kx[i], d);
#pragma unroll
        for (int o = 1; o < LPT; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const float s = valid ? d * p.scale : -INFINITY;
        if (s > m[g]) {
          const float corr = lse_factor(m[g], s);
          l[g] *= corr;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] *= corr;
          m[g] = s;
        }
        const float w = valid ? __expf(s - m[g]) : 0.f;
        l[g] += w;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(w, vx[i], acc[g][i]);
      }
    }
    __syncwarp();  // every lane is done with the slot before it is refilled
    if (lane == 0 && j + STAGES < nblk) issue(j + STAGES);
  }

  // merge the token groups of the warp
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o), lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float M = fmaxf(m[g], mo);
      const float fs = lse_factor(m[g], M), fo = lse_factor(mo, M);
      l[g] = l[g] * fs + lo * fo;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][i], o);
        acc[g][i] = acc[g][i] * fs + ao * fo;
      }
      m[g] = M;
    }
  }
  // The ring is free now (all copies were waited for): reuse its head as the cross-warp exchange buffer.
  __syncthreads();
  float* s_acc = reinterpret_cast<float*>(attn_smem);  // [warps][G][HD]
  if (tg == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s_acc[((size_t)warp * G + g) * HD + li * 4 + i] = acc[g][i];
        s_acc[((size_t)warp * G + g) * HD + (li + LPT) * 4 + i] = acc[g][4 + i];
      }
      if (li == 0) {
        s_m[warp][g] = m[g];
        s_l[warp][g] = l[g];
      }
    }
  }
  __syncthreads();
  pi_grid_launch_dependents();
  for (int idx = tid; idx < G * HD; idx += kAttnWarps * 32) {
    const int g = idx / HD, d = idx - g * HD;
    float M = s_m[0][g];
#pragma unroll
    for (int w = 1; w < kAttnWarps; ++w) M = fmaxf(M, s_m[w][g]);
    float ls = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float f = lse_factor(s_m[w][g], M);
      ls += s_l[w][g] * f;
      a += s_acc[((size_t)w * G + g) * HD + d] * f;
    }
    const int h = kvh * G + g;
    if (p.nsplit == 1) {
      p.out[(size_t)b * p.out_stride + (size_t)h * HD + d] = a * (1.0f / fmaxf(ls, 1e-12f));
    } else {
      const size_t slot = ((size_t)b * p.H + h) * p.nsplit + split;
      p.part_acc[slot * HD + d] = a;
      if (d == 0) {
        p.part_ml[slot * 2] = M;
        p.part_ml[slot * 2 + 1] = ls;
      }
    }
  }
}

// ---- block-size-16 kernel: tile-at-a-time softmax, packed f32x2 math ---------------------------------------
//
// Same staging as attn_decode_tma_kernel (per-warp TMA ring of K|V tiles), but the arithmetic is organised per
// 16-token tile instead of per token, which cuts the instruction count several times:
//   A. scores of all 16 tokens: each lane multiplies its 8 dims of K into the G query heads with packed
//      fma.rn.f32x2, then a reduce-scatter over the LPT lanes of the token (halving the value count at each
//      shuffle step) leaves every lane with the finished score of ONE (token, head);
//   B. one softmax update per tile: tile max per head, one correction factor, one exp per (token, head);
//   C. accumulation: the probabilities are broadcast back over the token's lanes and multiplied into V with
//      fma.rn.f32x2; the accumulator is rescaled only when some head's maximum actually moved.
// Scores are kept in the log2 domain (scale * log2(e) folded into one multiply, ex2.approx for the exponentials).
template <int HD, int G, int STAGES>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode_v3_kernel(const AttnParams p) {
  constexpr int BS = 16;
  constexpr int LPT = HD / 8;       // lanes per token
  constexpr int TPW = 32 / LPT;     // tokens per warp step
  constexpr int STEPS = BS / TPW;   // steps per tile
  constexpr uint32_t kTileBytes = 2u * BS * HD * sizeof(float);
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(128) unsigned char attn_smem[];
  __shared__ __align__(8) unsigned long long bars[kAttnWarps][STAGES];
  __shared__ float s_m[kAttnWarps][G], s_l[kAttnWarps][G];

  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tg = lane / LPT, li = lane % LPT;
  float* ring = reinterpret_cast<float*>(attn_smem) + (size_t)warp * STAGES * (kTileBytes / 4);

  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(attn_smem_u32(&bars[warp][s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  int lb_begin = split * p.blocks_per_cta;   // first logical block of this CTA (an entry without a window start)
  // physical block of this warp's tile j (lane 0 looks it up one tile ahead of the copy that needs it, so the
  // table read is not on the path between two tiles)
  auto lookup = [&](int j) { return p.tables[(size_t)b * p.max_blocks + lb_begin + warp + j * kAttnWarps]; };
  auto issue = [&](int j, int pb) {
    const float* src = p.kv + pi_kv_tile_offset(p.L, p.layer, pb, kvh, 0);
    const uint32_t bar = attn_smem_u32(&bars[warp][j % STAGES]);
    const uint32_t dst = attn_smem_u32(ring + (size_t)(j % STAGES) * (kTileBytes / 4));
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kTileBytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(kTileBytes), "r"(bar)
                 : "memory");
  };
  // Tiles of blocks that were complete when the batch was uploaded (everything below the entry's position then, for
  // an entry without a window start) do not depend on the kernel ahead of this one in the stream, and neither do the
  // block tables: the first copies of the ring go out before the dependency wait.  Such an entry starts at block 0,
  // so this CTA's range is known without reading the (device-updated) positions.
  const int len = p.lens[b];
  const int safe = p.safe_lb ? min(p.safe_lb[b], len) : 0;
  int npre = 0;
  if (lane == 0)
    for (; npre < STAGES && lb_begin + warp + npre * kAttnWarps < min(safe, lb_begin + p.blocks_per_cta); ++npre) issue(npre, lookup(npre));
  pi_grid_dependency_wait();

  const int pos = p.pos[b], st = p.start[b];
  const int lb_first = st / BS, lb_last = pos / BS;
  lb_begin = lb_first + split * p.blocks_per_cta;   // unchanged when anything was fetched early (then st == 0)
  const int lb_end = min(min(lb_last + 1, lb_begin + p.blocks_per_cta), len);
  const int nblk = (st <= pos && lb_begin + warp < lb_end) ? (lb_end - lb_begin - warp + kAttnWarps - 1) / kAttnWarps : 0;
  int pb_next = -1;
  if (lane == 0) {
    for (int j = npre; j < STAGES && j < nblk; ++j) issue(j, lookup(j));
    if (STAGES < nblk) pb_next = lookup(STAGES);
  }

  // q: 8 dims per lane (16-byte chunks li and li + LPT of the head) for every head of the group, as float2 pairs
  float2 qv[G][4];
  const float* qb = p.q + (size_t)b * p.q_stride + (size_t)kvh * G * HD;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float4 a = ldg_f4(qb + g * HD + li * 4), c = ldg_f4(qb + g * HD + (li + LPT) * 4);
    qv[g][0] = make_float2(a.x, a.y); qv[g][1] = make_float2(a.z, a.w);
    qv[g][2] = make_float2(c.x, c.y); qv[g][3] = make_float2(c.z, c.w);
  }
  float2 acc[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[g][i] = make_float2(0.f, 0.f);
  // softmax state of the head this lane owns (log2 domain), over the tokens of its token group
  float m_own = -INFINITY, l_own = 0.f;
  const float scale2 = p.scale * kLog2e;
  const int lane_base = lane & ~(LPT - 1);

  for (int j = 0; j < nblk; ++j) {
    const int slot = j % STAGES;
    const uint32_t bar = attn_smem_u32(&bars[warp][slot]);
    const uint32_t parity = (j / STAGES) & 1;
    uint32_t done = 0;
    for (uint32_t spin = 0; spin < kAttnSpinLimit && !done; ++spin)
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (!__all_sync(0xffffffffu, done != 0)) {
      if (lane == 0 && p.err_flag) atomicExch(p.err_flag, 7);
      for (int jj = j + 1; jj < nblk && jj < j + STAGES; ++jj) {  // bounded drain of the copies still in flight
        const uint32_t b2 = attn_smem_u32(&bars[warp][jj % STAGES]), par2 = (jj / STAGES) & 1;
        uint32_t d2 = 0;
        for (uint32_t spin = 0; spin < kAttnSpinLimit && !d2; ++spin)
          asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                       : "=r"(d2) : "r"(b2), "r"(par2) : "memory");
      }
      break;
    }
    const int lb = lb_begin + warp + j * kAttnWarps;
    const int t_lo = max(st - lb * BS, 0), t_hi = min(pos - lb * BS, BS - 1);
    const bool whole = (t_lo == 0) && (t_hi == BS - 1);
    const float* Kt = ring + (size_t)slot * (kTileBytes / 4);
    const float* Vt = Kt + BS * HD;

    // ---- A: scores -------------------------------------------------------------------------------------
    float sc[STEPS];
#pragma unroll
    for (int stp = 0; stp < STEPS; ++stp) {
      const int t = stp * TPW + tg;
      const float4 k0 = *reinterpret_cast<const float4*>(Kt + t * HD + li * 4);
      const float4 k1 = *reinterpret_cast<const float4*>(Kt + t * HD + (li + LPT) * 4);
      const float2 kk[4] = {make_float2(k0.x, k0.y), make_float2(k0.z, k0.w), make_float2(k1.x, k1.y), make_float2(k1.z, k1.w)};
      float vals[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float2 d = __fmul2_rn(qv[g][0], kk[0]);
        d = __ffma2_rn(qv[g][1], kk[1], d);
        d = __ffma2_rn(qv[g][2], kk[2], d);
        d = __ffma2_rn(qv[g][3], kk[3], d);
        vals[g] = d.x + d.y;
      }
      // reduce-scatter over the LPT lanes of the token: halve the value count per step while it is > 1
      int n = G;
#pragma unroll
      for (int o = 1; o < LPT; o <<= 1) {
        if (n > 1) {
          const int h = n >> 1;
          const bool up = (lane & o) != 0;
#pragma unroll
          for (int i = 0; i < G / 2; ++i) {
            if (i < h) {
              const float send = up ? vals[i] : vals[i + h];
              const float recv = __shfl_xor_sync(0xffffffffu, send, o);
              vals[i] = (up ? vals[i + h] : vals[i]) + recv;
            }
          }
          n = h;
        } else {
          vals[0] += __shfl_xor_sync(0xffffffffu, vals[0], o);
        }
      }
      const bool valid = whole || (t >= t_lo && t <= t_hi);
      sc[stp] = valid ? vals[0] * scale2 : -INFINITY;
    }

    // ---- B: one softmax update per tile ---------------------------------------------------------------------
    float tmax = sc[0];
#pragma unroll
    for (int stp = 1; stp < STEPS; ++stp) tmax = fmaxf(tmax, sc[stp]);
#pragma unroll
    for (int o = LPT; o < 32; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));  // across token groups
    const float m_new = fmaxf(m_own, tmax);
    const float corr = (m_own == -INFINITY) ? 1.f : ex2_approx(m_own - m_new);  // nothing accumulated yet: nothing to rescale
    float pr[STEPS];
    float psum = 0.f;
#pragma unroll
    for (int stp = 0; stp < STEPS; ++stp) {
      pr[stp] = (sc[stp] == -INFINITY) ? 0.f : ex2_approx(sc[stp] - m_new);
      psum += pr[stp];
    }
    l_own = l_own * corr + psum;
    m_own = m_new;

    // ---- C: accumulate ---------------------------------------------------------------------------------------
    if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float cg_ = __shfl_sync(0xffffffffu, corr, lane_base + attn_owner_lane<G, LPT>(g));
        const float2 c2 = make_float2(cg_, cg_);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[g][i] = __fmul2_rn(acc[g][i], c2);
      }
    }
#pragma unroll
    for (int stp = 0; stp < STEPS; ++stp) {
      const int t = stp * TPW + tg;
      float4 v0 = *reinterpret_cast<const float4*>(Vt + t * HD + li * 4);
      float4 v1 = *reinterpret_cast<const float4*>(Vt + t * HD + (li + LPT) * 4);
      if (!whole && !(t >= t_lo && t <= t_hi)) {  // never multiply a slot that was not written for this sequence
        v0 = make_float4(0.f, 0.f, 0.f, 0.f);
        v1 = v0;
      }
      const float2 vv[4] = {make_float2(v0.x, v0.y), make_float2(v0.z, v0.w), make_float2(v1.x, v1.y), make_float2(v1.z, v1.w)};
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pg = __shfl_sync(0xffffffffu, pr[stp], lane_base + attn_owner_lane<G, LPT>(g));
        const float2 p2 = make_float2(pg, pg);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[g][i] = __ffma2_rn(p2, vv[i], acc[g][i]);
      }
    }
    __syncwarp();
    if (lane == 0 && j + STAGES < nblk) {
      issue(j + STAGES, pb_next);
      if (j + 1 + STAGES < nblk) pb_next = lookup(j + 1 + STAGES);   // consumed one iteration from now
    }
  }

  // ---- merge the token groups of the warp (the owned head's m, l; every head's accumulator) -------------------
  // first bring every token group to the common maximum per head
  float m_all = m_own;
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
  const float f_own = (m_own == -INFINITY) ? 0.f : ex2_approx(m_own - m_all);
  float l_all = l_own * f_own;
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) l_all += __shfl_xor_sync(0xffffffffu, l_all, o);
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float fg = __shfl_sync(0xffffffffu, f_own, lane_base + attn_owner_lane<G, LPT>(g));
    const float2 f2 = make_float2(fg, fg);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 a = __fmul2_rn(acc[g][i], f2);
#pragma unroll
      for (int o = LPT; o < 32; o <<= 1) {
        a.x += __shfl_xor_sync(0xffffffffu, a.x, o);
        a.y += __shfl_xor_sync(0xffffffffu, a.y, o);
      }
      acc[g][i] = a;
    }
  }
  __syncthreads();  // every warp is done with its ring: reuse it for the cross-warp exchange
  float* s_acc = reinterpret_cast<float*>(attn_smem);  // [warps][G][HD]
  if (tg == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* dstp = s_acc + ((size_t)warp * G + g) * HD;
      *reinterpret_cast<float4*>(dstp + li * 4) = make_float4(acc[g][0].x, acc[g][0].y, acc[g][1].x, acc[g][1].y);
      *reinterpret_cast<float4*>(dstp + (li + LPT) * 4) = make_float4(acc[g][2].x, acc[g][2].y, acc[g][3].x, acc[g][3].y);
    }
    const int g_own = attn_owned_head<G, LPT>(li);
    if (attn_owner_lane<G, LPT>(g_own) == li) {  // one writer per head
      s_m[warp][g_own] = m_all;
      s_l[warp][g_own] = l_all;
    }
  }
  __syncthreads();
  pi_grid_launch_dependents();
  constexpr float kLn2 = 0.6931471805599453f;
  for (int idx = tid; idx < G * HD; idx += kAttnWarps * 32) {
    const int g = idx / HD, d = idx - g * HD;
    float M = s_m[0][g];
#pragma unroll
    for (int w = 1; w < kAttnWarps; ++w) M = fmaxf(M, s_m[w][g]);
    float ls = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float f = (s_m[w][g] == -INFINITY) ? 0.f : ex2_approx(s_m[w][g] - M);
      ls += s_l[w][g] * f;
      a += s_acc[((size_t)w * G + g) * HD + d] * f;
    }
    const int h = kvh * G + g;
    if (p.nsplit == 1) {
      p.out[(size_t)b * p.out_stride + (size_t)h * HD + d] = a * (1.0f / fmaxf(ls, 1e-12f));
    } else {
      const size_t slot = ((size_t)b * p.H + h) * p.nsplit + split;
      p.part_acc[slot * HD + d] = a;
      if (d == 0) {
        p.part_ml[slot * 2] = M * kLn2;  // the merge kernel works in the natural-log domain
        p.part_ml[slot * 2 + 1] = ls;
      }
    }
  }
}

// grid (H, B), HD threads (rounded up to a warp): merge the KV splits.
__global__ void attn_combine_kernel(const AttnParams p, int HD) {
  pi_grid_dependency_wait();
  const int h = blockIdx.x, b = blockIdx.y;
  const size_t base = ((size_t)b * p.H + h) * p.nsplit;
  float M = -INFINITY;
  for (int s = 0; s < p.nsplit; ++s) M = fmaxf(M, p.part_ml[(base + s) * 2]);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float ls = 0.f, a = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
      const float f = lse_factor(p.part_ml[(base + s) * 2], M);
      ls += p.part_ml[(base + s) * 2 + 1] * f;
      a += p.part_acc[(base + s) * HD + d] * f;
    }
    const float v = a * (1.0f / fmaxf(ls, 1e-12f));
    p.out[(size_t)b * p.out_stride + (size_t)h * HD + d] = v;
    if (p.emit_base) {
      unsigned short p0, p1, p2;
      pi_split3(v, p0, p1, p2);
      unsigned short* q = p.emit_base + (size_t)b * p.emit_k + (size_t)h * HD + d;
      q[0] = p0;
      q[p.emit_plane_stride] = p1;
      q[2 * p.emit_plane_stride] = p2;
    }
  }
}

// Any shape: one warp per (query head, entry); lane owns dims lane, lane+32, ...
constexpr int kGenericMaxPerLane = 16;
__global__ void __launch_bounds__(32) attn_generic_kernel(const AttnParams p, int HD, int group) {
  pi_grid_dependency_wait();
  const int h = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
  const int kvh = h / group, BS = p.L.block_size;
  const int pos = p.pos[b], st = p.start[b], len = p.lens[b];
  float qv[kGenericMaxPerLane], acc[kGenericMaxPerLane];
#pragma unroll
  for (int i = 0; i < kGenericMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < HD ? p.q[(size_t)b * p.q_stride + (size_t)h * HD + d] : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int t = st; t <= pos; ++t) {
    const int lb = t / BS;
    if (lb >= len) break;  // everything further is unmapped as well
    const int pb = p.tables[(size_t)b * p.max_blocks + lb];
    const float* K = p.kv + pi_kv_tile_offset(p.L, p.layer, pb, kvh, 0) + (size_t)(t - lb * BS) * HD;
    const float* V = K + (size_t)BS * HD;
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < kGenericMaxPerLane; ++i)
      if (lane + 32 * i < HD) d = fmaf(qv[i], K[lane + 32 * i], d);
    const float s = pi_warp_sum(d) * p.scale;
    if (s > m) {
      const float corr = m == -INFINITY ? 0.f : expf(m - s);
      l *= corr;
#pragma unroll
      for (int i = 0; i < kGenericMaxPerLane; ++i) acc[i] *= corr;
      m = s;
    }
    const float w = expf(s - m);
    l += w;
#pragma unroll
    for (int i = 0; i < kGenericMaxPerLane; ++i)
      if (lane + 32 * i < HD) acc[i] = fmaf(w, V[lane + 32 * i], acc[i]);
  }
  const float inv = 1.0f / fmaxf(l, 1e-12f);
#pragma unroll
  for (int i = 0; i < kGenericMaxPerLane; ++i)
    if (lane + 32 * i < HD) p.out[(size_t)b * p.out_stride + (size_t)h * HD + lane + 32 * i] = acc[i] * inv;
}

template <typename K, typename... Args>
cudaError_t launch_attn(pi_ctx* ctx, K kernel, dim3 grid, dim3 block, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <int HD>
cudaError_t launch_fast(pi_ctx* ctx, int group, dim3 grid, const AttnParams& p) {
  switch (group) {
    case 1: return launch_attn(ctx, attn_decode_kernel<HD, 1>, grid, dim3(kAttnWarps * 32), p);
    case 2: return launch_attn(ctx, attn_decode_kernel<HD, 2>, grid, dim3(kAttnWarps * 32), p);
    case 4: return launch_attn(ctx, attn_decode_kernel<HD, 4>, grid, dim3(kAttnWarps * 32), p);
    default: return launch_attn(ctx, attn_decode_kernel<HD, 8>, grid, dim3(kAttnWarps * 32), p);
  }
}

template <int HD, int G, int STAGES>
cudaError_t launch_tma_one(pi_ctx* ctx, dim3 grid, const AttnParams& p, size_t smem) {
  auto k = attn_decode_tma_kernel<HD, G, STAGES>;
  static pi_smem_grant granted;  // per instantiation: the attribute call is slow, so raise the limit only when needed
  if (smem > granted.of(ctx)) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    granted.of(ctx) = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kAttnWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, k, p);
}

template <int HD, int G, int STAGES>
cudaError_t launch_v3_one(pi_ctx* ctx, dim3 grid, const AttnParams& p, size_t smem) {
  auto k = attn_decode_v3_kernel<HD, G, STAGES>;
  static pi_smem_grant granted;
  if (smem > granted.of(ctx)) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    granted.of(ctx) = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kAttnWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, k, p);
}

template <int HD, int STAGES>
cudaError_t launch_v3(pi_ctx* ctx, int group, dim3 grid, const AttnParams& p, size_t smem) {
  switch (group) {
    case 1: return launch_v3_one<HD, 1, STAGES>(ctx, grid, p, smem);
    case 2: return launch_v3_one<HD, 2, STAGES>(ctx, grid, p, smem);
    case 4: return launch_v3_one<HD, 4, STAGES>(ctx, grid, p, smem);
    default: return launch_v3_one<HD, 8, STAGES>(ctx, grid, p, smem);
  }
}

template <int HD, int STAGES>
cudaError_t launch_tma(pi_ctx* ctx, int group, dim3 grid, const AttnParams& p, size_t smem) {
  switch (group) {
    case 1: return launch_tma_one<HD, 1, STAGES>(ctx, grid, p, smem);
    case 2: return launch_tma_one<HD, 2, STAGES>(ctx, grid, p, smem);
    case 4: return launch_tma_one<HD, 4, STAGES>(ctx, grid, p, smem);
    default: return launch_tma_one<HD, 8, STAGES>(ctx, grid, p, smem);
  }
}

}  // namespace

// Host block tables and per-entry metadata -> one device buffer, through pinned memory.
pi_status pi_upload_attn_batch(pi_ctx* ctx, const int32_t* tables_host, int max_blocks, const int32_t* lens_host,
                               const int32_t* pos_host, const int32_t* start_host, int B, int block_size, int num_blocks,
                               pi_attn_batch* out) {
  PI_REQUIRE(ctx, B > 0, "attention needs at least one entry");
  PI_REQUIRE(ctx, max_blocks >= 0 && block_size > 0, "bad block table shape");
  const int mb = std::max(max_blocks, 1);
  const size_t n = (size_t)B * mb + 4 * (size_t)B;
  PI_TRY(pi_reserve(ctx, &ctx->attn_tables, n * sizeof(int32_t)));
  PI_TRY(pi_reserve_pinned(ctx, n * sizeof(int32_t)));
  int32_t* h = static_cast<int32_t*>(ctx->pinned);
  int32_t* h_lens = h + (size_t)B * mb;
  int32_t* h_pos = h_lens + B;
  int32_t* h_start = h_pos + B;
  int32_t* h_safe = h_start + B;
  long total = 0;
  int widest = 0;
  bool shared = B > 1;
  for (int b = 0; b < B; ++b) {
    const int len = lens_host[b];
    if (shared && b > 0 &&
        (len != lens_host[0] || (len > 0 && memcmp(tables_host + (size_t)b * max_blocks, tables_host, (size_t)len * sizeof(int32_t)) != 0)))
      shared = false;
    PI_REQUIRE(ctx, len >= 0 && len <= max_blocks, "entry %d: table length %d outside [0, %d]", b, len, max_blocks);
    PI_REQUIRE(ctx, pos_host[b] >= 0 && start_host[b] >= 0, "entry %d: negative position", b);
    for (int i = 0; i < mb; ++i) h[(size_t)b * mb + i] = (i < len) ? tables_host[(size_t)b * max_blocks + i] : -1;
    h_lens[b] = len;
    h_pos[b] = pos_host[b];
    h_start[b] = start_host[b];
    h_safe[b] = 0;
    if (start_host[b] <= pos_host[b]) {
      const int nb = pos_host[b] / block_size - start_host[b] / block_size + 1;
      total += nb;
      widest = std::max(widest, nb);
    }
  }
  // Which leading blocks of an entry may be fetched before the K/V writes of this step have landed: those below its
  // position that no entry of the batch writes in this step (an entry writes the block that holds its position; several
  // positions of one sequence in one batch - a prefill chunk, a speculative group - write blocks that the others read).
  if (num_blocks > 0) {
    std::vector<uint8_t>& written = ctx->scratch_block_marks;
    written.assign((size_t)num_blocks, 0);
    for (int b = 0; b < B; ++b) {
      const int lb = pos_host[b] / block_size;
      if (lb < lens_host[b]) {
        const int32_t pb = tables_host[(size_t)b * max_blocks + lb];
        if (pb >= 0 && pb < num_blocks) written[pb] = 1;
      }
    }
    for (int b = 0; b < B; ++b) {
      if (start_host[b] != 0) continue;
      const int limit = std::min(pos_host[b] / block_size, lens_host[b]);
      int lb = 0;
      for (; lb < limit; ++lb) {
        const int32_t pb = tables_host[(size_t)b * max_blocks + lb];
        if (pb < 0 || pb >= num_blocks || written[pb]) break;
      }
      h_safe[b] = lb;
    }
  }
  int32_t* d = static_cast<int32_t*>(ctx->attn_tables.ptr);
  PI_CUDA(ctx, cudaMemcpyAsync(d, h, n * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
  out->tables = d;
  out->max_blocks = mb;
  out->lens = d + (size_t)B * mb;
  out->pos = out->lens + B;
  out->start = out->pos + B;
  out->safe_lb = out->start + B;
  out->B = B;
  out->max_window_blocks = widest;
  out->total_window_blocks = total;
  out->shared_table = shared;
  out->shared_len = shared ? lens_host[0] : 0;
  return PI_OK;
}

pi_status pi_launch_attention(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q,
                              size_t q_stride, float* out, size_t out_stride, const pi_attn_batch& batch,
                              pi_act_planes* emit, bool* emitted) {
  if (emitted) *emitted = false;
  const pi_kv_layout& L = pool->L;
  PI_REQUIRE(ctx, layer >= 0 && layer < L.num_layers, "layer %d outside the pool's %d layers", layer, L.num_layers);
  PI_REQUIRE(ctx, L.num_kv_heads > 0 && num_heads % L.num_kv_heads == 0 && num_heads > 0,
             "num_attention_heads (%d) must be a multiple of num_key_value_heads (%d)", num_heads, L.num_kv_heads);
  const int group = num_heads / L.num_kv_heads, HD = L.head_dim;
  AttnParams p;
  p.q = q;
  p.q_stride = q_stride;
  p.out = out;
  p.out_stride = out_stride;
  p.kv = pool->data;
  p.L = L;
  p.layer = layer;
  p.H = num_heads;
  p.tables = batch.tables;
  p.max_blocks = batch.max_blocks;
  p.lens = batch.lens;
  p.pos = batch.pos;
  p.start = batch.start;
  p.safe_lb = batch.safe_lb;
  p.scale = 1.0f / sqrtf((float)HD);
  p.err_flag = ctx->dev_err;
  p.nsplit = 1;
  p.blocks_per_cta = std::max(batch.max_window_blocks, 1);
  p.part_ml = nullptr;
  p.part_acc = nullptr;
  p.emit_base = nullptr;
  p.emit_plane_stride = 0;
  p.emit_k = 0;

  pi_prof_scope prof(ctx, PI_PROF_ATTENTION);
  if (pi_attention_shared_usable(ctx, pool, num_heads, q, q_stride, out, out_stride, batch))
    return pi_launch_attention_shared(ctx, pool, layer, num_heads, q, q_stride, out, out_stride, batch);
  const bool fast = (HD == 64 || HD == 128) && (group == 1 || group == 2 || group == 4 || group == 8) &&
                    ((uintptr_t)q % 16 == 0) && (q_stride % 4 == 0);
  if (fast && batch.flat_warps > 0 && ((uintptr_t)out % 16 == 0) && (out_stride % 4 == 0))
    return pi_launch_attention_flat(ctx, pool, layer, num_heads, q, q_stride, out, out_stride, batch, emit, emitted);
  cudaError_t e;
  if (!fast) {
    PI_REQUIRE(ctx, HD <= 32 * kGenericMaxPerLane, "head_dim %d is not supported (max %d)", HD, 32 * kGenericMaxPerLane);
    e = launch_attn(ctx, attn_generic_kernel, dim3(num_heads, batch.B), dim3(32), p, HD, group);
    if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
    ctx->launches++;
    return PI_OK;
  }

  // Split the KV axis so that about four CTAs per SM stream the pool.
  const long pairs_blocks = batch.total_window_blocks * L.num_kv_heads;
  const long target_ctas = (long)ctx->sm_count * 4;
  int bpc = (int)((pairs_blocks + target_ctas - 1) / target_ctas);
  bpc = std::max(bpc, kAttnWarps);
  bpc = (bpc + kAttnWarps - 1) / kAttnWarps * kAttnWarps;
  int nsplit = (std::max(batch.max_window_blocks, 1) + bpc - 1) / bpc;
  if (nsplit > 64) {
    nsplit = 64;
    bpc = (batch.max_window_blocks + nsplit - 1) / nsplit;
  }
  // Windows of up to 12 blocks whose merge kernel would have nothing else to do (no planes to emit): one CTA per
  // (kv head, entry) walks the whole window and writes the output itself - one launch less per layer (measured at
  // batch 1: faster up to about 190 tokens of context, slower from 300 on).
  if (!(emit && emit->base) && batch.max_window_blocks <= 12) {
    nsplit = 1;
    bpc = (std::max(batch.max_window_blocks, 1) + kAttnWarps - 1) / kAttnWarps * kAttnWarps;
  }
  p.blocks_per_cta = bpc;
  p.nsplit = nsplit;
  if (nsplit > 1) {
    const size_t slots = (size_t)batch.B * num_heads * nsplit;
    PI_TRY(pi_reserve(ctx, &ctx->attn_partial, slots * (HD + 2) * sizeof(float)));
    p.part_acc = static_cast<float*>(ctx->attn_partial.ptr);
    p.part_ml = p.part_acc + slots * HD;
  }
  const dim3 grid(L.num_kv_heads, batch.B, nsplit);
  // Tiles staged through shared memory by bulk copies when a ring of them fits; direct loads otherwise.
  const size_t tile_bytes = 2 * (size_t)L.block_size * HD * sizeof(float);
  const int stages = HD == 64 ? 3 : 2;
  const size_t ring_bytes = (size_t)kAttnWarps * stages * tile_bytes;
  if (ctx->opt_attn_tma == 1 && L.block_size == 16)
    e = HD == 64 ? launch_v3<64, 3>(ctx, group, grid, p, ring_bytes) : launch_v3<128, 2>(ctx, group, grid, p, ring_bytes);
  else if (ctx->opt_attn_tma && tile_bytes % 16 == 0 && ring_bytes + 4096 <= ctx->smem_optin && tile_bytes < (1u << 20))
    e = HD == 64 ? launch_tma<64, 3>(ctx, group, grid, p, ring_bytes) : launch_tma<128, 2>(ctx, group, grid, p, ring_bytes);
  else
    e = HD == 64 ? launch_fast<64>(ctx, group, grid, p) : launch_fast<128>(ctx, group, grid, p);
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  if (nsplit > 1) {
    if (emit && emit->base && emit->K == num_heads * HD) {
      p.emit_base = reinterpret_cast<unsigned short*>(emit->base);
      p.emit_plane_stride = emit->plane_stride;
      p.emit_k = emit->K;
      emit->row_scale = nullptr;
      emit->sumsq_tiles = 0;
      if (emitted) *emitted = true;
    }
    e = launch_attn(ctx, attn_combine_kernel, dim3(num_heads, batch.B), dim3(HD), p, HD);
    if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "attention combine launch failed: %s", cudaGetErrorString(e));
    ctx->launches++;
  }
  return PI_OK;
}
