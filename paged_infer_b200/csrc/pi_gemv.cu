// Dequantising GEMV / small-batch GEMM on CUDA cores, and the row quantiser.
//
// y[m][r] = scale[r] * sum_k W[r][k] * x[m][k] with W int8 (or bf16 / f32 with
// scale 1), x f32, f32 accumulation.  This is the decode-sized path: every
// weight byte is read from HBM exactly once per launch with 128-bit loads.
//
// The grid is persistent (a couple of CTAs per SM).  Each CTA stages the
// activations into shared memory once with a bulk async copy (TMA,
// cp.async.bulk), optionally applies RMSNorm to them there, and stores them in a
// layout that makes the later 128-bit reads conflict-free.  Each warp then walks
// row pairs; its weight loads are issued a group of 4 steps (2 KiB per row) at a
// time and one group ahead of the arithmetic, so that enough bytes are in flight
// to cover the HBM latency and a DRAM page is visited once.  int8 is widened
// with a byte permute into the mantissa of 2^23 (no quarter-rate I2F); products
// use packed fma.rn.f32x2; rows are reduced with shuffles.  Epilogues: store,
// residual add, or SwiGLU over interleaved gate/up rows.
//
// Replaces math::matvec_i8_weight_parallel / matmat_i8_weight_parallel and the
// f32 twins (reference src/math.rs:93-275, :473-512) and math::quantize_rows_i8
// (:456-469).
#include <algorithm>

#include "pi_common.cuh"

namespace {

constexpr int kRows = 2;    // output rows per warp pass
constexpr int kSteps = 4;   // 512-byte steps of a row per load group
constexpr int kSplitWarps = 3;   // warps that share a row pair when a matrix has few, long rows
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ int4 ld_stream_16(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// 16 bytes of weights -> EPL floats, as float2 pairs.
template <typename WT>
struct Widen;
template <>
struct Widen<int8_t> {
  static constexpr int EPL = 16;
  // int8 -> f32 without the quarter-rate I2F: flip the sign bit so the byte is
  // b+128 in [0,255], drop it into the mantissa of 2^23, subtract 2^23+128.
  __device__ static __forceinline__ void run(const int4& v, float2* f) {
    const uint32_t w[4] = {(uint32_t)v.x ^ 0x80808080u, (uint32_t)v.y ^ 0x80808080u, (uint32_t)v.z ^ 0x80808080u,
                           (uint32_t)v.w ^ 0x80808080u};
    const float2 bias = make_float2(-8388736.0f, -8388736.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = make_float2(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7440)),
                                   __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7441)));
      const float2 b = make_float2(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7442)),
                                   __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7443)));
      f[2 * i + 0] = __fadd2_rn(a, bias);
      f[2 * i + 1] = __fadd2_rn(b, bias);
    }
  }
};
template <>
struct Widen<uint16_t> {  // bf16 bits
  static constexpr int EPL = 8;
  __device__ static __forceinline__ void run(const int4& v, float2* f) {
    const uint32_t w[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
  }
};
template <>
struct Widen<float> {
  static constexpr int EPL = 4;
  __device__ static __forceinline__ void run(const int4& v, float2* f) {
    f[0] = make_float2(__int_as_float(v.x), __int_as_float(v.y));
    f[1] = make_float2(__int_as_float(v.z), __int_as_float(v.w));
  }
};

struct GemvParams {
  const void* W;
  const float* scales;
  const float* x;
  float* out;
  const float* norm_weight;
  size_t ld, x_stride, out_stride;
  int N, K, M;
  float eps;
  int use_tma;
  int* err_flag;
  // optional: rotary embedding + KV write for the fused [q;k;v] projection (rope_hd = 0: off).  The two rows of a
  // warp's pair are then the two members of a rotation pair, so the finished pair can be rotated in registers.
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

// Row r (0 or 1) of row pair `pair`: consecutive rows, or the members of a rotation pair of one head.
template <bool ROPE>
__device__ __forceinline__ int gemv_row(const GemvParams& p, int pair, int r) {
  if (!ROPE) return pair * kRows + r;
  const int half = p.rope_hd >> 1, head = pair / half, j = pair - head * half;
  return p.rope_style == 0 ? head * p.rope_hd + j + r * half : head * p.rope_hd + 2 * j + r;
}

// A lane reads U = EPL/4 consecutive 16-byte units of x per step.  Stored
// linearly that is a U-way bank conflict for 128-bit shared loads, so unit j of
// lane-group g lives at slot j ^ s(g): every quarter warp then touches eight
// distinct 16-byte bank groups.
template <int U>
__device__ __forceinline__ int unit_swizzle(int group) {
  if (U == 4) return (group >> 1) & 3;
  if (U == 2) return (group >> 2) & 1;
  return 0;
}

// KS > 1 (matrices with few, long rows): KS consecutive warps share a row pair, warp ks of them takes the K groups
// ks, ks + KS, ...; the partial sums meet in shared memory and are added in warp order by the first warp of the set.
template <typename WT, int MB, int EPI, bool NORM, bool ROPE, int KS = 1>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvParams p) {
  constexpr int EPL = Widen<WT>::EPL;
  constexpr int U = EPL / 4;
  constexpr int kStepElems = 32 * EPL;
  constexpr int kGroupElems = kSteps * kStepElems;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  float* xs = reinterpret_cast<float*>(smem_raw);  // [MB][ld]
  __shared__ __align__(8) unsigned long long mbar;
  __shared__ float red[MB][8];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int ld = (int)p.ld, K = p.K;
  const int m0 = blockIdx.y * MB;
  const int mcount = min(MB, p.M - m0);
  const int npairs = (p.N + kRows - 1) / kRows;
  const int ngroups = (ld + kGroupElems - 1) / kGroupElems;
  const int total_warps = gridDim.x * nwarps;
  const int k_lane = lane * EPL;

  // Work items of this warp: (row pair, K group), row pairs strided by the number of warps in the grid.
  int4 wcur[kSteps][kRows], wnxt[kSteps][kRows];
  auto load_group = [&](int4 (&g)[kSteps][kRows], int pair, int kg) {
    const unsigned char* rowp[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r)
      rowp[r] = reinterpret_cast<const unsigned char*>(p.W) + (size_t)min(gemv_row<ROPE>(p, pair, r), p.N - 1) * ld * sizeof(WT);
#pragma unroll
    for (int t = 0; t < kSteps; ++t) {
      const int k = kg * kGroupElems + t * kStepElems + k_lane;
#pragma unroll
      for (int r = 0; r < kRows; ++r) g[t][r] = (k < ld) ? ld_stream_16(rowp[r] + (size_t)k * sizeof(WT)) : make_int4(0, 0, 0, 0);
    }
  };
  __shared__ float part[2][KS > 1 ? 8 : 1][kRows][MB];   // KS > 1: partial sums of the warps of a set (two parities)
  const int ks = KS > 1 ? warp % KS : 0;
  const int pair_stride = KS > 1 ? total_warps / KS : total_warps;
  int pair = KS > 1 ? (blockIdx.x * nwarps + warp) / KS : blockIdx.x * nwarps + warp, kg = ks;
  int n_done = 0;
  // the first group does not depend on the producer kernel: request it before waiting for the activations
  if (pair < npairs) load_group(wcur, pair, kg);
  // so does the norm weight of the group this thread will scale first (K a multiple of 4: no ragged tail)
  float4 nw_pre[U];
  const bool nw_pre_ok = NORM && (K & 3) == 0;
  if (nw_pre_ok) {
    const int groups = ld / EPL, g = tid % groups;
#pragma unroll
    for (int j = 0; j < U; ++j)
      nw_pre[j] = (tid < groups * MB && g * EPL + 4 * j < K) ? __ldg(reinterpret_cast<const float4*>(p.norm_weight + (size_t)g * EPL) + j)
                                                              : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  pi_grid_dependency_wait();

  // fused [q;k;v] projection: lane m finishes activation row m0+m; its position and the physical block that takes its
  // K and V are looked up now, off the path between the dot products and the stores
  int my_pos = 0, my_pb = -1;
  if (ROPE && lane < mcount) {
    const int gm = m0 + lane;
    my_pos = p.pos[gm];
    const int lb = my_pos / p.L.block_size;
    if (lb < p.lens[gm]) my_pb = p.tables[(size_t)gm * p.max_blocks + lb];
  }

  // ---- stage x[m0 .. m0+mcount) into shared memory, once per CTA ---------------------------------
  bool landed = false;
  if (p.use_tma) {
    if (tid == 0) {
      const uint32_t bar = smem_u32(&mbar);
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      const uint32_t bytes = (uint32_t)(mcount * K * sizeof(float));
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
      for (int m = 0; m < mcount; ++m) {
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                smem_u32(xs + (size_t)m * ld)),
            "l"(p.x + (size_t)(m0 + m) * p.x_stride), "r"((uint32_t)(K * sizeof(float))), "r"(bar)
            : "memory");
      }
    }
    // zero the padding and the unused batch rows (disjoint from the copy's bytes)
    for (int m = 0; m < MB; ++m) {
      const int from = (m < mcount) ? K : 0;
      for (int k = from + tid; k < ld; k += blockDim.x) xs[(size_t)m * ld + k] = 0.f;
    }
    __syncthreads();  // barrier initialised before anyone polls it
    const uint32_t bar = smem_u32(&mbar);
    uint32_t done = 0;
    for (uint32_t spin = 0; spin < kSpinLimit && !done; ++spin) {
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(done)
          : "r"(bar), "r"(0u)
          : "memory");
    }
    landed = __syncthreads_and((int)done) != 0;
    if (!landed && tid == 0 && p.err_flag) atomicExch(p.err_flag, 1);  // bulk copy never completed: reload below
  }
  if (!landed) {
    for (int m = 0; m < MB; ++m) {
      const float* src = p.x + (size_t)(m0 + m) * p.x_stride;
      for (int k = tid; k < ld; k += blockDim.x) xs[(size_t)m * ld + k] = (m < mcount && k < K) ? src[k] : 0.f;
    }
    __syncthreads();
  }

  // ---- in-place pass per EPL-float group: swizzle units; with RMSNorm (math::rms_norm, src/math.rs:4-22) also
  // multiply by the norm weight and collect the sum of squares.  The row factor 1/rms is applied to the finished
  // dot products in the epilogue (one pass and two barriers less than normalising x first).
  {
    const int groups = ld / EPL;
    float ssm[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) ssm[m] = 0.f;
    for (int idx = tid; idx < groups * MB; idx += blockDim.x) {
      const int m = idx / groups, g = idx - m * groups;
      float4* base = reinterpret_cast<float4*>(xs + (size_t)m * ld + (size_t)g * EPL);
      float4 u[U];
#pragma unroll
      for (int j = 0; j < U; ++j) u[j] = base[j];
      if (NORM) {
        float sq = 0.f;
#pragma unroll
        for (int j = 0; j < U; ++j) {
          sq = fmaf(u[j].x, u[j].x, sq);
          sq = fmaf(u[j].y, u[j].y, sq);
          sq = fmaf(u[j].z, u[j].z, sq);
          sq = fmaf(u[j].w, u[j].w, sq);
        }
#pragma unroll
        for (int mm = 0; mm < MB; ++mm) ssm[mm] += (mm == m) ? sq : 0.f;
        const float4* nw = reinterpret_cast<const float4*>(p.norm_weight + (size_t)g * EPL);
#pragma unroll
        for (int j = 0; j < U; ++j) {
          const int kk = g * EPL + 4 * j;
          float4 w4 = (nw_pre_ok && idx == tid) ? nw_pre[j] : (kk + 3 < K) ? nw[j] : make_float4(0.f, 0.f, 0.f, 0.f);
          if (kk < K && kk + 3 >= K) {  // ragged tail of the norm weight
            w4.x = p.norm_weight[kk];
            w4.y = kk + 1 < K ? p.norm_weight[kk + 1] : 0.f;
            w4.z = kk + 2 < K ? p.norm_weight[kk + 2] : 0.f;
            w4.w = 0.f;
          }
          u[j].x *= w4.x;
          u[j].y *= w4.y;
          u[j].z *= w4.z;
          u[j].w *= w4.w;
        }
      }
      const int s = unit_swizzle<U>(g & 31);
#pragma unroll
      for (int j = 0; j < U; ++j) base[j ^ s] = u[j];
    }
    if (NORM) {
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        const float ss = pi_warp_sum(ssm[m]);
        if (lane == 0) red[m][warp] = ss;
      }
    }
    __syncthreads();
  }
  // 1/rms of activation row m, from the warps' partial sums in warp order (every thread gets the same bits)
  auto row_factor = [&](int m) -> float {
    if (!NORM) return 1.0f;
    float ss = 0.f;
    for (int w = 0; w < nwarps; ++w) ss += red[m][w];
    return 1.0f / sqrtf(ss / (float)K + p.eps);
  };
  pi_grid_launch_dependents();

  // ---- stream the weight rows -------------------------------------------------
  float2 acc[kRows][MB];  // even / odd partial sums
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[r][m] = make_float2(0.f, 0.f);

  const int s = unit_swizzle<U>(lane);
  while (pair < npairs) {
    int npair = pair, nkg = kg + KS;
    if (nkg >= ngroups) {
      nkg = ks;
      npair = pair + pair_stride;
    }
    if (npair < npairs) load_group(wnxt, npair, nkg);
    // residual add: the value this lane will add to is requested before the arithmetic of the pair's last group
    float old_out = 0.f;
    if (EPI == PI_EPI_ADD && !ROPE && ks == 0 && kg + KS >= ngroups) {
      const int r = lane / MB, m = lane - r * MB;
      if (r < kRows && m < mcount && pair * kRows + r < p.N)
        old_out = p.out[(size_t)(m0 + m) * p.out_stride + pair * kRows + r];
    }
    float sc[kRows] = {1.0f, 1.0f};   // the rows' scales, requested likewise
    if (kg + KS >= ngroups && ks == 0) {
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const int rw = gemv_row<ROPE>(p, pair, r);
        if (p.scales && rw < p.N) sc[r] = p.scales[rw];
      }
    }
    float rp_cs = 1.f, rp_sn = 0.f;   // rotation of this pair at lane m's position, requested likewise
    if (ROPE && lane < mcount && kg + KS >= ngroups) {
      const int half = p.rope_hd >> 1;
      rp_cs = p.rope_cos[(size_t)my_pos * half + pair % half];
      rp_sn = p.rope_sin[(size_t)my_pos * half + pair % half];
    }

    const int kbase = kg * kGroupElems;
#pragma unroll
    for (int t = 0; t < kSteps; ++t) {
      if (kbase + t * kStepElems >= ld) break;  // uniform across the warp
      const int k0 = kbase + t * kStepElems + k_lane;
      if (k0 < ld) {
        float2 wf[kRows][EPL / 2];
#pragma unroll
        for (int r = 0; r < kRows; ++r) Widen<WT>::run(wcur[t][r], wf[r]);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          const float4* xb = reinterpret_cast<const float4*>(xs + (size_t)m * ld + k0);
#pragma unroll
          for (int j = 0; j < U; ++j) {
            const float4 xv = xb[j ^ s];
            const float2 xlo = make_float2(xv.x, xv.y), xhi = make_float2(xv.z, xv.w);
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
              acc[r][m] = __ffma2_rn(wf[r][2 * j + 0], xlo, acc[r][m]);
              acc[r][m] = __ffma2_rn(wf[r][2 * j + 1], xhi, acc[r][m]);
            }
          }
        }
      }
    }

    if (kg + KS >= ngroups) {  // this warp's share of the row pair is complete: reduce, apply the scale, write
      const int row0 = pair * kRows;
      float tot[kRows][MB];
#pragma unroll
      for (int r = 0; r < kRows; ++r)
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          tot[r][m] = pi_warp_sum(acc[r][m].x + acc[r][m].y);
          acc[r][m] = make_float2(0.f, 0.f);
        }
      bool writer = true;
      if (KS > 1) {
        // the warps of the set meet at their own named barrier (they walk the same row pairs, so they arrive the same
        // number of times); the first warp adds the partial sums in warp order
        const int par = n_done & 1;
        ++n_done;
        if (lane == 0) {
#pragma unroll
          for (int r = 0; r < kRows; ++r)
#pragma unroll
            for (int m = 0; m < MB; ++m) part[par][warp][r][m] = tot[r][m];
        }
        asm volatile("bar.sync %0, %1;" ::"r"(1 + warp / KS), "r"(KS * 32) : "memory");
        writer = ks == 0;
        if (writer) {
#pragma unroll
          for (int r = 0; r < kRows; ++r)
#pragma unroll
            for (int m = 0; m < MB; ++m) {
              float t = part[par][warp][r][m];
#pragma unroll
              for (int j = 1; j < KS; ++j) t += part[par][warp + j][r][m];
              tot[r][m] = t;
            }
        }
      }
      if (writer) {
      if (ROPE) {
        // fused [q;k;v] projection: lane m finishes activation row m0+m - rotate the pair (q and k rows), leave q in
        // `out`, scatter k and v into the pool at the row's position (skipped when the block is not mapped)
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          if (lane == m && m < mcount) {
            const int gm = m0 + m, hd = p.rope_hd;
            const int ra = gemv_row<ROPE>(p, pair, 0), rb = gemv_row<ROPE>(p, pair, 1);
            const int seg = ra < p.rope_q_rows ? 0 : (ra < p.rope_q_rows + p.rope_kv_rows ? 1 : 2);
            const int within = ra - (seg == 0 ? 0 : (seg == 1 ? p.rope_q_rows : p.rope_q_rows + p.rope_kv_rows));
            const float rf = row_factor(m);
            float a = tot[0][m] * sc[0] * rf, c = tot[1][m] * sc[1] * rf;
            if (seg < 2) {
              const float na = a * rp_cs - c * rp_sn, nc = c * rp_cs + a * rp_sn;
              a = na;
              c = nc;
            }
            float* o = p.out + (size_t)gm * p.out_stride;
            o[ra] = a;
            o[rb] = c;
            if (seg > 0) {
              const int off = my_pos % p.L.block_size;
              if (my_pb >= 0) {   // an unmapped position: the write is skipped silently
                const int pb = my_pb;
                const int kh = within / hd, da = within - kh * hd;
                float* dst = p.kv + pi_kv_tile_offset(p.L, p.layer, pb, kh, seg == 2 ? 1 : 0) + (size_t)off * hd;
                dst[da] = a;
                dst[da + (rb - ra)] = c;
              }
            }
          }
        }
      } else if (EPI == PI_EPI_SWIGLU) {
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          if (lane == m && m < mcount && row0 + 1 < p.N) {
            const float rf = row_factor(m);
            const float g = tot[0][m] * sc[0] * rf, u = tot[1][m] * sc[1] * rf;
            p.out[(size_t)(m0 + m) * p.out_stride + (row0 >> 1)] = (g / (1.0f + expf(-g))) * u;
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < kRows; ++r)
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            if (lane == r * MB + m && m < mcount && row0 + r < p.N) {
              float* o = p.out + (size_t)(m0 + m) * p.out_stride + row0 + r;
              const float v = tot[r][m] * sc[r] * row_factor(m);
              *o = (EPI == PI_EPI_ADD) ? (old_out + v) : v;
            }
          }
      }
      }  // writer
    }
#pragma unroll
    for (int t = 0; t < kSteps; ++t)
#pragma unroll
      for (int r = 0; r < kRows; ++r) wcur[t][r] = wnxt[t][r];
    pair = npair;
    kg = nkg;
  }
}

template <typename WT, int MB>
cudaError_t launch_gemv_t(pi_ctx* ctx, const GemvParams& p, int epi, bool norm, dim3 grid, int threads, size_t smem,
                          bool pdl, int ksplit) {
  void (*k)(const GemvParams) = nullptr;
#define PI_PICK(E, Nrm) k = gemv_kernel<WT, MB, E, Nrm, false>
  if (ksplit == kSplitWarps) {   // few long rows (pi_launch_gemv asks for it only without norm, rotary embedding, SwiGLU)
    if (epi == PI_EPI_ADD) k = gemv_kernel<WT, MB, PI_EPI_ADD, false, false, kSplitWarps>;
    else k = gemv_kernel<WT, MB, PI_EPI_STORE, false, false, kSplitWarps>;
  } else if (epi == PI_EPI_STORE && p.rope_hd) {   // fused [q;k;v] projection: own instantiation, the others stay as they are
    if (norm) k = gemv_kernel<WT, MB, PI_EPI_STORE, true, true>; else k = gemv_kernel<WT, MB, PI_EPI_STORE, false, true>;
  } else if (epi == PI_EPI_STORE) {
    if (norm) PI_PICK(PI_EPI_STORE, true); else PI_PICK(PI_EPI_STORE, false);
  } else if (epi == PI_EPI_ADD) {
    if (norm) PI_PICK(PI_EPI_ADD, true); else PI_PICK(PI_EPI_ADD, false);
  } else {
    if (norm) PI_PICK(PI_EPI_SWIGLU, true); else PI_PICK(PI_EPI_SWIGLU, false);
  }
#undef PI_PICK
  static pi_smem_grant granted;  // per instantiation of this launcher; attribute calls are slow
  if (smem > std::max(granted.of(ctx), (size_t)48 * 1024)) {
    // the launcher covers several kernel variants: raise the limit on all of them at once
    for (auto kk : {gemv_kernel<WT, MB, PI_EPI_STORE, true, false>, gemv_kernel<WT, MB, PI_EPI_STORE, false, false>,
                    gemv_kernel<WT, MB, PI_EPI_ADD, true, false>, gemv_kernel<WT, MB, PI_EPI_ADD, false, false>,
                    gemv_kernel<WT, MB, PI_EPI_SWIGLU, true, false>, gemv_kernel<WT, MB, PI_EPI_SWIGLU, false, false>,
                    gemv_kernel<WT, MB, PI_EPI_STORE, true, true>, gemv_kernel<WT, MB, PI_EPI_STORE, false, true>,
                    gemv_kernel<WT, MB, PI_EPI_ADD, false, false, kSplitWarps>,
                    gemv_kernel<WT, MB, PI_EPI_STORE, false, false, kSplitWarps>}) {
      cudaError_t e = cudaFuncSetAttribute(kk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
    }
    granted.of(ctx) = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, k, p);
}

template <typename WT>
cudaError_t launch_gemv_w(pi_ctx* ctx, const GemvParams& p, int mb, int epi, bool norm, dim3 grid, int threads,
                          size_t smem, bool pdl, int ksplit) {
  switch (mb) {
    case 1: return launch_gemv_t<WT, 1>(ctx, p, epi, norm, grid, threads, smem, pdl, ksplit);
    case 2: return launch_gemv_t<WT, 2>(ctx, p, epi, norm, grid, threads, smem, pdl, ksplit);
    default: return launch_gemv_t<WT, 4>(ctx, p, epi, norm, grid, threads, smem, pdl, ksplit);
  }
}

// ---- quantiser ---------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float* __restrict__ w, size_t w_ld, int cols,
                                                            int8_t* __restrict__ q, size_t q_ld,
                                                            float* __restrict__ scales) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const size_t row = blockIdx.x;
  const float* src = w + row * w_ld;
  float m = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, fabsf(src[c]));  // fmaxf drops NaN like f32::max
  m = pi_warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) mm = fmaxf(mm, red[i]);
    const float scale = mm > 0.f ? __fdiv_rn(mm, 127.0f) : 1.0f;
    s_scale = scale;
    scales[row] = scale;
  }
  __syncthreads();
  const float scale = s_scale;
  int8_t* dst = q + row * q_ld;
  for (int c = threadIdx.x; c < (int)q_ld; c += blockDim.x) {
    int8_t code = 0;
    if (c < cols) {
      const float v = roundf(__fdiv_rn(src[c], scale));  // half away from zero, true division
      // Rust's clamp keeps NaN and `as i8` maps it to 0; fminf/fmaxf would drop the NaN instead.
      code = (v != v) ? (int8_t)0 : (int8_t)(int)fminf(fmaxf(v, -127.0f), 127.0f);
    }
    dst[c] = code;  // padding columns are zero
  }
}

}  // namespace

pi_status pi_launch_quantize(pi_ctx* ctx, const float* w_dev, size_t w_ld, size_t rows, size_t cols, int8_t* q_dev,
                             size_t q_ld, float* scales_dev) {
  if (rows == 0) return PI_OK;
  quantize_rows_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(w_dev, w_ld, (int)cols, q_dev, q_ld, scales_dev);
  PI_CHECK_LAUNCH(ctx);
  return PI_OK;
}

bool pi_gemv_can_rope(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, const pi_rope_kv& r) {
  (void)ctx;
  if (a.epi != PI_EPI_STORE || a.emit || !r.pool || !r.batch || !r.rope_cos || !r.rope_sin) return false;
  if (r.head_dim < 2 || (r.head_dim & 1)) return false;               // an odd head_dim leaves one element unpaired
  if (r.pool->L.head_dim != r.head_dim || r.pool->L.num_kv_heads != r.num_kv_heads) return false;
  if (lin->rows != (size_t)(r.num_heads + 2 * r.num_kv_heads) * r.head_dim) return false;
  return r.style == 0 || r.style == 1;
}

pi_status pi_launch_gemv(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a) {
  PI_REQUIRE(ctx, a.M >= 1, "projection batch must be at least 1");
  PI_REQUIRE(ctx, a.epi != PI_EPI_SWIGLU || lin->rows % 2 == 0, "SwiGLU epilogue needs interleaved gate/up rows");
  if (lin->rows == 0) return PI_OK;
  int mb = a.M >= 4 ? 4 : a.M >= 2 ? 2 : 1;
  while (mb > 1 && (size_t)mb * lin->ld * sizeof(float) > ctx->smem_optin - 2048) mb >>= 1;
  const size_t smem = (size_t)mb * lin->ld * sizeof(float);
  PI_REQUIRE(ctx, smem <= ctx->smem_optin - 2048, "projection input of %zu columns does not fit shared memory", lin->cols);

  // Persistent grid: two CTAs of up to 8 warps per SM; narrower CTAs when there are few row pairs, so that
  // every SM still gets work.
  const size_t npairs = (lin->rows + kRows - 1) / kRows;
  const int mtiles = (a.M + mb - 1) / mb;
  const size_t max_ctas = std::max<size_t>(1, (size_t)ctx->sm_count * 2 / mtiles);
  int warps = 8;
  while (warps > 1 && (npairs + warps - 1) / warps < max_ctas) warps >>= 1;
  size_t ctas = std::min<size_t>((npairs + warps - 1) / warps, max_ctas);
  // Few rows of at least three 2 KiB groups each, with no prologue or pairing to keep (the down projection of a small
  // model): at most half the warps of the grid would find a row pair, each walking its groups one after the other.
  // Sets of three warps share a row pair instead: three times the loads in flight.
  int ksplit = 1;
  const size_t row_bytes = lin->ld * (lin->kind == PI_INT8 ? 1 : lin->kind == PI_BF16 ? 2 : 4);
  if (!a.norm_weight && !a.rope && a.epi != PI_EPI_SWIGLU && row_bytes > (size_t)(kSplitWarps - 1) * kSteps * 512 &&
      npairs * 2 <= max_ctas * 8) {
    ksplit = kSplitWarps;
    warps = 2 * kSplitWarps;
    ctas = std::min<size_t>((npairs + 1) / 2, max_ctas);
  }
  dim3 grid((unsigned)ctas, (unsigned)mtiles);

  GemvParams p;
  p.W = lin->w;
  p.scales = lin->kind == PI_INT8 ? lin->scales : nullptr;
  p.x = a.x;
  p.out = a.out;
  p.norm_weight = a.norm_weight;
  p.ld = lin->ld;
  p.x_stride = a.x_stride;
  p.out_stride = a.out_stride;
  p.N = (int)lin->rows;
  p.K = (int)lin->cols;
  p.M = a.M;
  p.eps = a.norm_eps;
  p.err_flag = ctx->dev_err;
  p.rope_hd = 0;
  if (a.rope) {
    const pi_rope_kv& r = *a.rope;
    PI_REQUIRE(ctx, pi_gemv_can_rope(ctx, lin, a, r), "this launch cannot fold the rotary embedding and the KV write in");
    p.rope_hd = r.head_dim;
    p.rope_q_rows = r.num_heads * r.head_dim;
    p.rope_kv_rows = r.num_kv_heads * r.head_dim;
    p.rope_style = r.style;
    p.rope_cos = r.rope_cos;
    p.rope_sin = r.rope_sin;
    p.kv = r.pool->data;
    p.L = r.pool->L;
    p.layer = r.layer;
    p.tables = r.batch->tables;
    p.max_blocks = r.batch->max_blocks;
    p.lens = r.batch->lens;
    p.pos = r.batch->pos;
  }
  p.use_tma = ((lin->cols * sizeof(float)) % 16 == 0) && ((uintptr_t)a.x % 16 == 0) &&
              ((a.x_stride * sizeof(float)) % 16 == 0) && ((size_t)mb * lin->cols * sizeof(float) < (1u << 20));
  const bool norm = a.norm_weight != nullptr;
  pi_prof_scope prof(ctx, PI_PROF_GEMV);
  cudaError_t e;
  if (lin->kind == PI_INT8)
    e = launch_gemv_w<int8_t>(ctx, p, mb, a.epi, norm, grid, warps * 32, smem, ctx->opt_pdl, ksplit);
  else if (lin->kind == PI_BF16)
    e = launch_gemv_w<uint16_t>(ctx, p, mb, a.epi, norm, grid, warps * 32, smem, ctx->opt_pdl, ksplit);
  else
    e = launch_gemv_w<float>(ctx, p, mb, a.epi, norm, grid, warps * 32, smem, ctx->opt_pdl, ksplit);
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "gemv launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  return PI_OK;
}
