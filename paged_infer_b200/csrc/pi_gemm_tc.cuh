// Device side of the tcgen05 dequant GEMM (pi_gemm_tc.cu): mbarrier / TMEM / MMA wrappers in inline PTX, the exact
// int8 -> bf16 widening, the launch parameters of one projection and its epilogues (store / residual add / SwiGLU,
// planes for the next projection, rotary embedding + KV write).
#pragma once

#include <cuda.h>

#include "pi_common.cuh"

namespace pi_tc {

constexpr int kBM = 128;            // weight rows per CTA (MMA M)
constexpr int kBK = 128;            // K elements per pipeline stage (two 128-byte swizzle atoms of 16-bit elements)
constexpr int kProducerWarps = 16;  // stream + widen the weights; all of them emit the result
constexpr int kParkWarps = 8;       // warps 0-7 also move the accumulator from TMEM to shared memory
constexpr int kThreads = (kProducerWarps + 2) * 32;
constexpr uint32_t kSpinLimit = 1u << 21;
constexpr int kPlanes = 3;
constexpr int kACols = kBK / 2;     // 128 bf16 of a weight row = 64 32-bit TMEM columns
// Every CTA asks for all 512 TMEM columns and for at least this much shared memory, so two of these CTAs never share
// an SM: a CTA blocked in tcgen05.alloc while its cluster peers wait for it at a cluster barrier could deadlock.
constexpr size_t kMinSmem = 120 * 1024;

struct GemmParams {
  const int8_t* W;
  const float* scales;      // [N]
  float* out;
  size_t ld, out_stride;
  int N, K, M;
  int ksplit, nkb;          // K splits, total K blocks
  int epi;
  int n_out_also;           // plain store epilogue: the result also goes to these bases (other ranks' memory)
  float* out_also[8];
  int* err_flag;
  // row factor of the activations: given, or derived from partial sums of squares, or 1
  const float* act_scale;   // [M]
  const float* sumsq_in;    // [sumsq_tiles][sumsq_stride]
  int sumsq_tiles;
  size_t sumsq_stride;
  float eps;
  // optional: the result as planes for the next projection
  __nv_bfloat16* emit_base; // [3][.][emit_k]
  size_t emit_plane_stride;
  int emit_k;
  const float* emit_norm;   // [emit_k] or null
  float* emit_sumsq;        // [row tiles][emit_sumsq_stride] or null
  size_t emit_sumsq_stride;
  // optional: rotary embedding + KV write for the fused [q;k;v] projection (rope_hd = 0: off)
  int rope_hd, rope_q_rows, rope_kv_rows, rope_style;
  const float* rope_cos;
  const float* rope_sin;
  float* kv;
  pi_kv_layout L;
  int layer;
  const int32_t* tables;
  int max_blocks;
  const int32_t* lens;
  const int32_t* pos;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// The same, for kernels that start before the kernel ahead of them in the stream has finished (programmatic dependent
// launch): polls are only counted once `*dep_ok` says that this launch's dependency is resolved.  Until then nothing
// here can make progress and the wait is the preceding kernel's, however long that runs - it must not be mistaken for
// a wait of this kernel that ran out.
__device__ __forceinline__ bool mbar_wait_dep(uint32_t bar, uint32_t parity, const volatile int* dep_ok) {
  for (uint32_t spin = 0; spin < kSpinLimit;) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if (*dep_ok) ++spin;
  }
  return false;
}

__device__ __forceinline__ void ld_stream_32(const void* p, uint32_t* v) {
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "l"(p));
}

// 4 int8 -> 4 bf16 (exact): byte b^0x80 into the mantissa of 2^23 as f32, minus (2^23 + 128); an integer of at
// most 8 significant bits has a zero low half as f32, so its upper 16 bits are the bf16 value.
__device__ __forceinline__ void widen4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t x = w ^ 0x80808080u;
  const float2 f01 = make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650)),
                                 __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7651)));
  const float2 f23 = make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7652)),
                                 __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7653)));
  const float2 bias = make_float2(-8388736.0f, -8388736.0f);
  const float2 a = __fadd2_rn(f01, bias), b = __fadd2_rn(f23, bias);
  lo = __byte_perm(__float_as_uint(a.x), __float_as_uint(a.y), 0x7632);
  hi = __byte_perm(__float_as_uint(b.x), __float_as_uint(b.y), 0x7632);
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);       // start address
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset
  d |= (uint64_t)1 << 46;                       // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
  return d;
}

// D[tmem_d] (+)= A[tmem_a] * B[smem descriptor]
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// Columns [c, c+16) of the three accumulator groups of this thread's lane, added.
template <int BN>
__device__ __forceinline__ void tmem_ld_sum16(uint32_t lane_base, int c, float* v) {
  uint32_t a[16], b[16], d[16];
  tmem_ld16_issue(lane_base + (uint32_t)c, a);
  tmem_ld16_issue(lane_base + (uint32_t)(BN + c), b);
  tmem_ld16_issue(lane_base + (uint32_t)(2 * BN + c), d);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = (__uint_as_float(a[i]) + __uint_as_float(b[i])) + __uint_as_float(d[i]);
}

// 16 consecutive TMEM columns of this thread's lane (lane = 32 * (warp % 4) + laneid).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

__device__ __forceinline__ void split3(float y, unsigned short& p0, unsigned short& p1, unsigned short& p2) { pi_split3(y, p0, p1, p2); }

// Epilogue of the fused [q;k;v] projection: thread = four adjacent output columns rr..rr+3 of activation row m,
// all 32 lanes of the warp on the same m (so the shuffles below are safe).  Row tiles are whole heads: the NeoX
// partner (j, j + hd/2) of a lane's four values sits in lane ^ (hd/8), interleaved pairs (2j, 2j+1) are the
// thread's own.  q: rotated into out.  k: rotated into out and into the pool.  v: copied into the pool.
__device__ __forceinline__ void emit_rope(const GemmParams& p, int m, int rr, int lane, float v0, float v1, float v2, float v3) {
  const int hd = p.rope_hd, half = hd >> 1;
  const bool valid = m < p.M && rr < p.N;
  const int mm = valid ? m : 0;
  const int seg = rr < p.rope_q_rows ? 0 : (rr < p.rope_q_rows + p.rope_kv_rows ? 1 : 2);   // q, k, v
  const int within = rr - (seg == 0 ? 0 : (seg == 1 ? p.rope_q_rows : p.rope_q_rows + p.rope_kv_rows));
  const int d = within % hd;             // first of this thread's four dims inside its head
  const int position = p.pos[mm];
  float r[4] = {v0, v1, v2, v3};
  if (p.rope_style == 0) {
    const int plane = hd >> 3;            // partner lane distance
    const float o0 = __shfl_xor_sync(0xffffffffu, v0, plane), o1 = __shfl_xor_sync(0xffffffffu, v1, plane);
    const float o2 = __shfl_xor_sync(0xffffffffu, v2, plane), o3 = __shfl_xor_sync(0xffffffffu, v3, plane);
    if (seg < 2) {
      const int j = d % half;
      const float4 cs = __ldg(reinterpret_cast<const float4*>(p.rope_cos + (size_t)position * half + j));
      const float4 sn = __ldg(reinterpret_cast<const float4*>(p.rope_sin + (size_t)position * half + j));
      if (d < half) {    // this thread holds a = x[j..], the partner c = x[j + half..]:  a' = a*cos - c*sin
        r[0] = v0 * cs.x - o0 * sn.x; r[1] = v1 * cs.y - o1 * sn.y; r[2] = v2 * cs.z - o2 * sn.z; r[3] = v3 * cs.w - o3 * sn.w;
      } else {           // this thread holds c, the partner a:  c' = c*cos + a*sin
        r[0] = v0 * cs.x + o0 * sn.x; r[1] = v1 * cs.y + o1 * sn.y; r[2] = v2 * cs.z + o2 * sn.z; r[3] = v3 * cs.w + o3 * sn.w;
      }
    }
  } else if (seg < 2) {  // interleaved pairs (d, d+1), (d+2, d+3) with angles d/2, d/2 + 1
    const int j = d >> 1;
    const float c0 = __ldg(p.rope_cos + (size_t)position * half + j), s0 = __ldg(p.rope_sin + (size_t)position * half + j);
    const float c1 = __ldg(p.rope_cos + (size_t)position * half + j + 1), s1 = __ldg(p.rope_sin + (size_t)position * half + j + 1);
    r[0] = v0 * c0 - v1 * s0; r[1] = v1 * c0 + v0 * s0;
    r[2] = v2 * c1 - v3 * s1; r[3] = v3 * c1 + v2 * s1;
  }
  if (!valid) return;
  *reinterpret_cast<float4*>(p.out + (size_t)m * p.out_stride + rr) = make_float4(r[0], r[1], r[2], r[3]);
  if (seg == 0) return;
  const int lb = position / p.L.block_size, off = position % p.L.block_size;
  if (lb >= p.lens[m]) return;             // unmapped: the write is skipped silently
  const int pb = p.tables[(size_t)m * p.max_blocks + lb];
  const int kh = within / hd;
  float* dst = p.kv + pi_kv_tile_offset(p.L, p.layer, pb, kh, seg == 2 ? 1 : 0) + (size_t)off * hd + d;
  *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
}


// ---- the epilogue of one thread: four adjacent weight rows (= output columns) rr..rr+3 of one row tile -----------
// What the thread needs from global memory besides the accumulator: its rows' scales and, when the result is also
// emitted as planes for a following RMS-normalised projection, the norm weights of its columns.  Fetched early.
struct EpiRows {
  int rr;           // first of the four output columns
  float wsc[4];     // weight-row scales
  float nw[4];      // norm weights of the emitted planes (1 when there are none)
};

__device__ __forceinline__ void epi_rows_load(const GemmParams& p, int row0, int tid, EpiRows& e) {
  e.rr = row0 + (tid & 31) * 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    e.wsc[i] = (e.rr + i < p.N) ? __ldg(p.scales + e.rr + i) : 0.f;
    e.nw[i] = 1.0f;
  }
  if (p.emit_base && p.emit_norm) {
    if (p.epi == PI_EPI_SWIGLU) {
      if ((e.rr >> 1) + 1 < p.emit_k) {
        e.nw[0] = __ldg(p.emit_norm + (e.rr >> 1));
        e.nw[1] = __ldg(p.emit_norm + (e.rr >> 1) + 1);
      }
    } else if (e.rr + 3 < p.emit_k) {
#pragma unroll
      for (int i = 0; i < 4; ++i) e.nw[i] = __ldg(p.emit_norm + e.rr + i);
    }
  }
}

// One activation row m of the thread's four columns: acc = the raw dot products (all K, all planes added), `as` the
// row factor of the activations.  All 32 lanes of a warp call this with the same m (the rotary path and the sum of
// squares shuffle across the warp).  `tile` is the row tile (index of the per-tile sums of squares).  The residual
// is read past L1: inside a persistent kernel another SM may have written it a moment ago.
__device__ __forceinline__ void epi_row(const GemmParams& p, const EpiRows& e, int tile, int m, float as, float4 acc, int lane) {
  const int rr = e.rr;
  if (p.rope_hd) {   // fused [q;k;v] projection: rotary embedding + KV write
    emit_rope(p, m, rr, lane, acc.x * e.wsc[0] * as, acc.y * e.wsc[1] * as, acc.z * e.wsc[2] * as, acc.w * e.wsc[3] * as);
    return;
  }
  float sq = 0.f;
  if (m < p.M && rr < p.N) {
    const float v0 = acc.x * e.wsc[0] * as;
    const float v1 = acc.y * e.wsc[1] * as;
    const float v2 = acc.z * e.wsc[2] * as;
    const float v3 = acc.w * e.wsc[3] * as;
    if (p.epi == PI_EPI_SWIGLU) {
      float* o = p.out + (size_t)m * p.out_stride + (rr >> 1);
      const float s0 = silu_mul(v0, v1), s1 = silu_mul(v2, v3);
      if (rr + 1 < p.N) o[0] = s0;
      if (rr + 3 < p.N) o[1] = s1;
      if (p.emit_base && rr + 3 < p.N) {   // two adjacent columns = one 32-bit store per plane
        unsigned short a0, b0, c0, a1, b1, c1;
        split3(s0 * e.nw[0], a0, b0, c0);
        split3(s1 * e.nw[1], a1, b1, c1);
        uint32_t* q = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned short*>(p.emit_base) + (size_t)m * p.emit_k + (rr >> 1));
        q[0] = (uint32_t)a0 | ((uint32_t)a1 << 16);
        q[p.emit_plane_stride / 2] = (uint32_t)b0 | ((uint32_t)b1 << 16);
        q[p.emit_plane_stride] = (uint32_t)c0 | ((uint32_t)c1 << 16);
      }
    } else {
      float* o = p.out + (size_t)m * p.out_stride + rr;
      const bool add = p.epi == PI_EPI_ADD;
      float r[4] = {v0, v1, v2, v3};
      const bool full = rr + 3 < p.N;
      if (full && ((p.out_stride & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0)) {
        if (add) {
          const float4 old = __ldcg(reinterpret_cast<const float4*>(o));
          r[0] += old.x; r[1] += old.y; r[2] += old.z; r[3] += old.w;
        }
        *reinterpret_cast<float4*>(o) = make_float4(r[0], r[1], r[2], r[3]);
        for (int i = 0; i < p.n_out_also; ++i)   // tensor-parallel push: posted stores into the peers' buffers
          *reinterpret_cast<float4*>(p.out_also[i] + (size_t)m * p.out_stride + rr) = make_float4(r[0], r[1], r[2], r[3]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (rr + i < p.N) {
            if (add) r[i] += __ldcg(o + i);
            o[i] = r[i];
          } else {
            r[i] = 0.f;
          }
      }
      if (p.emit_base && full) {          // four adjacent columns = one 64-bit store per plane
        unsigned short a[4], b[4], c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) split3(r[i] * e.nw[i], a[i], b[i], c[i]);
        uint2* q = reinterpret_cast<uint2*>(reinterpret_cast<unsigned short*>(p.emit_base) + (size_t)m * p.emit_k + rr);
        q[0] = make_uint2((uint32_t)a[0] | ((uint32_t)a[1] << 16), (uint32_t)a[2] | ((uint32_t)a[3] << 16));
        q[p.emit_plane_stride / 4] = make_uint2((uint32_t)b[0] | ((uint32_t)b[1] << 16), (uint32_t)b[2] | ((uint32_t)b[3] << 16));
        q[p.emit_plane_stride / 2] = make_uint2((uint32_t)c[0] | ((uint32_t)c[1] << 16), (uint32_t)c[2] | ((uint32_t)c[3] << 16));
      }
      sq = fmaf(r[0], r[0], fmaf(r[1], r[1], fmaf(r[2], r[2], r[3] * r[3])));
    }
  }
  if (p.emit_sumsq) {   // sum over the 128 rows of this tile for activation row m, fixed order
    sq = pi_warp_sum(sq);
    if (lane == 0 && m < p.M) p.emit_sumsq[(size_t)tile * p.emit_sumsq_stride + m] = sq;
  }
}

// Row factor of activation row m: given, or 1/rms from the per-tile partial sums of squares (added in tile order), or 1.
__device__ __forceinline__ float act_row_factor(const GemmParams& p, int m) {
  float f = 1.0f;
  if (m < p.M) {
    if (p.act_scale) {
      f = __ldcg(p.act_scale + m);
    } else if (p.sumsq_in) {
      float t = 0.f;
      for (int i = 0; i < p.sumsq_tiles; ++i) t += __ldcg(p.sumsq_in + (size_t)i * p.sumsq_stride + m);
      f = 1.0f / sqrtf(t / (float)p.K + p.eps);
    }
  }
  return f;
}


// ---- host side (pi_gemm_tc.cu) ----------------------------------------------------------------------------------
// Activation rows per CTA tile: 16, 32 or 64.
int pick_bn(int M);
// Everything a launch of one projection needs: the parameter block and the tensor map over the activation planes
// ({K, M rows, 3 planes}; rows past M read as zero).  Also fills in what `a.emit` hands to the next projection.
pi_status build_gemm_params(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, const pi_act_planes& in, int BN,
                            GemmParams* p, CUtensorMap* map);

}  // namespace pi_tc
