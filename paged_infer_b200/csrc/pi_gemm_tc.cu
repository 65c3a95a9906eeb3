// Tensor-core dequant GEMM for batched decode and prefill: tcgen05.mma with the
// accumulator in tensor memory (TMEM), for int8 weights and f32 activations.
//
//   out[m][r] = scale[r] * sum_k W[r][k] * x[m][k]
//
// Swap-AB: the 128 weight rows of a CTA sit on the MMA's M axis, the batch on
// its N axis (16..128 per CTA).  The int8 weight tile is widened to fp16 (exact)
// in registers and written to shared memory in the 128-byte-swizzled K-major
// layout the MMA reads.  Each f32 activation is split into fp16 hi + fp16 lo
// after a power-of-two row scaling (x*s = hi + lo up to 2^-25 of the row's
// largest element); both planes are fetched by TMA (cp.async.bulk.tensor, no
// multicast) and the tile gets two MMAs per K step, which keeps the result
// f32-equivalent: every product is exact and accumulation is in f32.
//
// Warp roles (10 warps): 0-7 stream + widen the weights and later run the
// epilogue out of TMEM; warp 8 issues the TMA loads of the activations; warp 9
// allocates TMEM and issues the MMAs.  Stages are handed over with mbarriers;
// every wait is bounded and a wait that runs out raises the context's error
// word instead of hanging.
//
// K is split across CTAs when there are too few row tiles to fill the SMs; the
// K slices of one row tile form a thread-block cluster and add their partial
// tiles through distributed shared memory in rank order, so results do not
// depend on timing.
//
// Replaces math::matmat_i8_weight_parallel + transpose_rb_to_br for batches
// beyond a few rows (reference src/math.rs:223-290).
#include <cooperative_groups.h>
#include <cuda.h>
#include <stdlib.h>

#include <algorithm>

#include "pi_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kBM = 128;            // weight rows per CTA (MMA M)
constexpr int kBK = 128;            // K elements per pipeline stage (two 128-byte swizzle atoms of fp16)
constexpr int kProducerWarps = 8;
constexpr int kThreads = (kProducerWarps + 2) * 32;
constexpr uint32_t kSpinLimit = 1u << 21;
constexpr int kATileBytes = kBM * kBK * 2;  // 32 KiB of fp16 per stage

struct GemmParams {
  const int8_t* W;
  const float* scales;      // [N]
  const float* act_scale;   // [M] power-of-two factors to multiply back
  float* out;
  size_t ld, out_stride;
  int N, K, M;
  int ksplit, nkb;          // K splits, total K blocks
  int epi;
  int* err_flag;
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

__device__ __forceinline__ int4 ld_stream_16(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// 4 int8 -> 4 fp16 (exact): byte b^0x80 into the mantissa of 1024.0, minus 1152.
__device__ __forceinline__ void widen4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t x = w ^ 0x80808080u;
  const uint32_t a = __byte_perm(x, 0x64646464u, 0x4140);
  const uint32_t b = __byte_perm(x, 0x64646464u, 0x4342);
  const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));  // 1152.0
  __half2 ha = __hsub2(*reinterpret_cast<const __half2*>(&a), bias);
  __half2 hb = __hsub2(*reinterpret_cast<const __half2*>(&b), bias);
  lo = *reinterpret_cast<uint32_t*>(&ha);
  hi = *reinterpret_cast<uint32_t*>(&hb);
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

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with the accumulate flag fixed to 1 (no predicate set-up per instruction).
__device__ __forceinline__ void umma_f16_acc(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

// One output value through the epilogue.  SwiGLU pairs (gate, up) sit in adjacent rows = adjacent lanes.
__device__ __forceinline__ void emit(const GemmParams& p, int m, int row, float v, int lane) {
  if (p.epi == PI_EPI_SWIGLU) {
    const float other = __shfl_xor_sync(0xffffffffu, v, 1);
    if (!(lane & 1) && m < p.M && row + 1 < p.N) p.out[(size_t)m * p.out_stride + (row >> 1)] = silu_mul(v, other);
  } else if (m < p.M && row < p.N) {
    float* o = p.out + (size_t)m * p.out_stride + row;
    *o = (p.epi == PI_EPI_ADD) ? (*o + v) : v;
  }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap map_hi, const __grid_constant__ CUtensorMap map_lo) {
  constexpr int kBTileBytes = 2 * BN * 128;                 // one plane, two swizzle atoms
  constexpr int kStageBytes = kATileBytes + 2 * kBTileBytes;
  constexpr int kTmemCols = BN < 32 ? 32 : BN;              // power of two >= 32
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bars[2 * STAGES + 1];
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row0 = blockIdx.x * kBM, m0 = blockIdx.z * BN;
  const int kb_begin = (int)((long)blockIdx.y * p.nkb / p.ksplit), kb_end = (int)((long)(blockIdx.y + 1) * p.nkb / p.ksplit);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), accum_bar = smem_u32(&bars[2 * STAGES]);
  // Every thread releases the dependent grid right away (the release only happens once all threads of all CTAs
  // have done so): the next kernels then sit resident, with their own prologue done, by the time this one ends.
  pi_grid_launch_dependents();

  // ---- weight producers (warps 0-7): 16 KiB of int8 per stage, 4 x 16 bytes per thread ----------------------
  // chunk c = i*256 + tid covers row c/8, bytes (c%8)*16..+16 of the stage's 128 K elements.
  // Loads are issued a GROUP of kGroup K blocks at a time (512 contiguous bytes of every row), one group ahead
  // of the one being widened: 64 KiB in flight per CTA.  The first group is requested before anything else in
  // the kernel - weights never depend on the preceding kernel - so barrier set-up and the TMEM allocation hide
  // behind its latency.
  constexpr int kGroup = 4;
  const unsigned char* src[4];
  uint32_t dst[4];
  int4 cur[kGroup][4], nxt[kGroup][4];
  auto load_group = [&](int4 (&g)[kGroup][4], int kb0) {
#pragma unroll
    for (int d = 0; d < kGroup; ++d)
      if (kb0 + d < kb_end) {
#pragma unroll
        for (int i = 0; i < 4; ++i) g[d][i] = ld_stream_16(src[i] + (size_t)(kb0 + d) * kBK);
      }
  };
  if (warp < kProducerWarps) {
    const unsigned char* wbase = reinterpret_cast<const unsigned char*>(p.W);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = i * 256 + tid, r = c >> 3, kc = c & 7;
      const int row = min(row0 + r, p.N - 1);
      src[i] = wbase + (size_t)row * p.ld + kc * 16;
      // 16 int8 -> 32 bytes of fp16 = chunks 2*(kc&3), 2*(kc&3)+1 of atom kc>>2, XOR-swizzled by the row
      dst[i] = (uint32_t)((kc >> 2) * (kBM * 128) + r * 128) | ((uint32_t)(r & 7) << 16) | ((uint32_t)(kc & 3) << 24);
    }
    load_group(cur, kb_begin);
  }

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, kProducerWarps + 1);       // one arrival per producer warp + the TMA thread's expect_tx
      mbar_init(empty0 + 8 * s, 1);                        // one tcgen05.commit
    }
    mbar_init(accum_bar, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kProducerWarps + 1) {  // TMEM allocation is warp-wide
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;
  const uint32_t smem_base = smem_u32(smem);

  if (warp < kProducerWarps) {
    bool stop = false;
    for (int kb0 = kb_begin; kb0 < kb_end && !stop; kb0 += kGroup) {
      if (kb0 + kGroup < kb_end) load_group(nxt, kb0 + kGroup);
#pragma unroll
      for (int d = 0; d < kGroup; ++d) {
        const int kb = kb0 + d;
        if (kb >= kb_end || stop) break;
        const int it = kb - kb_begin, s = it % STAGES;
        // lane 0 polls for the whole warp: 256 threads hammering one mbarrier cost more than the copy itself
        int ok = 1;
        if (lane == 0) ok = (!s_abort && mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1)) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0 && !s_abort) {
            s_abort = 1;
            if (p.err_flag) atomicExch(p.err_flag, 2);
          }
          stop = true;
          break;
        }
        const uint32_t a_stage = smem_base + s * kStageBytes;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t h[8];
          widen4((uint32_t)cur[d][i].x, h[0], h[1]);
          widen4((uint32_t)cur[d][i].y, h[2], h[3]);
          widen4((uint32_t)cur[d][i].z, h[4], h[5]);
          widen4((uint32_t)cur[d][i].w, h[6], h[7]);
          const uint32_t rowbase = a_stage + (dst[i] & 0xFFFF), sw = (dst[i] >> 16) & 7, c0 = ((dst[i] >> 24) & 3) * 2;
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(rowbase + ((c0 ^ sw) << 4)), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(rowbase + (((c0 + 1) ^ sw) << 4)), "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * s);
      }
#pragma unroll
      for (int d = 0; d < kGroup; ++d)
#pragma unroll
        for (int i = 0; i < 4; ++i) cur[d][i] = nxt[d][i];
    }
    pi_grid_dependency_wait();  // the epilogue below touches memory the producer kernel may still be writing
  } else if (warp == kProducerWarps) {
    // ---- activation loader: TMA, hi and lo planes, two 64-column boxes each ---------------------------
    if (lane == 0) {
      pi_grid_dependency_wait();  // the activation planes come from the preceding kernel
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int it = kb - kb_begin, s = it % STAGES;
        if (s_abort) break;
        if (!mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1)) {
          s_abort = 1;
          if (p.err_flag) atomicExch(p.err_flag, 3);
          break;
        }
        const uint32_t bar = full0 + 8 * s;
        const uint32_t b_stage = smem_base + s * kStageBytes + kATileBytes;
        mbar_arrive_expect_tx(bar, 2 * kBTileBytes);
#pragma unroll
        for (int plane = 0; plane < 2; ++plane) {
          const CUtensorMap* map = plane == 0 ? &map_hi : &map_lo;
#pragma unroll
          for (int atom = 0; atom < 2; ++atom) {
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                    b_stage + plane * kBTileBytes + atom * (BN * 128)),
                "l"(map), "r"(bar), "r"(kb * kBK + atom * 64), "r"(m0)
                : "memory");
          }
        }
      }
    }
  } else {
    // ---- MMA issuer ------------------------------------------------------------------------------------------
    if (lane == 0) {
      // kind::f16, D = f32, A and B = f16, both K-major, N = BN, M = 128
      const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int it = kb - kb_begin, s = it % STAGES;
        if (s_abort || !mbar_wait(full0 + 8 * s, (it / STAGES) & 1)) {
          if (!s_abort && p.err_flag) atomicExch(p.err_flag, 4);
          s_abort = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // This one thread issues every MMA of the CTA, so its instruction count per K block bounds the whole
        // pipeline: the three descriptors of a stage are built once and only their start-address field (low
        // word, 16-byte units) is bumped by compile-time constants per MMA.
        const uint32_t a_stage = smem_base + s * kStageBytes;
        const uint64_t da0 = smem_desc(a_stage), dh0 = smem_desc(a_stage + kATileBytes), dl0 = smem_desc(a_stage + kATileBytes + kBTileBytes);
#pragma unroll
        for (int atom = 0; atom < 2; ++atom) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {  // 16 K elements = 32 bytes per MMA
            const uint64_t da = da0 + (uint64_t)((atom * (kBM * 128) + ks * 32) >> 4);
            const uint64_t dh = dh0 + (uint64_t)((atom * (BN * 128) + ks * 32) >> 4);
            const uint64_t dl = dl0 + (uint64_t)((atom * (BN * 128) + ks * 32) >> 4);
            if (atom == 0 && ks == 0) umma_f16(tmem, da, dh, idesc, kb > kb_begin ? 1u : 0u);
            else umma_f16_acc(tmem, da, dh, idesc);
            umma_f16_acc(tmem, da, dl, idesc);
          }
        }
        umma_commit(empty0 + 8 * s);  // the stage is free once these MMAs have read it
      }
      if (ok) umma_commit(accum_bar);
    }
  }

  // ---- epilogue: warps 0-7 read the accumulator (warp w owns TMEM lanes 32*(w%4).., columns split in halves) ----
  bool have_acc = false;
  if (warp < kProducerWarps) {
    int got = 0;
    if (lane == 0) {
      got = ((kb_begin < kb_end) && !s_abort && mbar_wait(accum_bar, 0)) ? 1 : 0;
      if (kb_begin < kb_end && !got && !s_abort) {
        s_abort = 1;
        if (p.err_flag) atomicExch(p.err_flag, 5);
      }
    }
    have_acc = __shfl_sync(0xffffffffu, got, 0) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  const int quad = warp & 3, half = warp >> 2;
  const int row = row0 + quad * 32 + lane;
  constexpr int kColsPerHalf = BN / 2 >= 16 ? BN / 2 : 16;  // BN 16: only the first half works
  const bool epi_warp = warp < kProducerWarps && (BN >= 32 || half == 0);

  if (p.ksplit == 1) {
    if (epi_warp && have_acc) {
      const float ws = row < p.N ? p.scales[row] : 0.f;
#pragma unroll 1
      for (int c0 = half * kColsPerHalf; c0 < (half + 1) * kColsPerHalf && c0 < BN; c0 += 16) {
        float v[16];
        tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + c0 + j;
          const float as = m < p.M ? p.act_scale[m] : 0.f;
          emit(p, m, row, v[j] * ws * as, lane);
        }
      }
    }
  } else {
    // K was split over the CTAs of a thread-block cluster (cluster rank = K slice).  Every CTA parks its raw
    // partial tile in its own shared memory (the pipeline stages are free by now), the cluster synchronises,
    // and each CTA then adds up and emits 1/ksplit of the tile's columns, reading its peers' tiles through
    // distributed shared memory in rank order - so the sum does not depend on timing.
    cg::cluster_group cluster = cg::this_cluster();
    float* my_part = reinterpret_cast<float*>(smem);  // [BN][128]
    if (epi_warp) {
#pragma unroll 1
      for (int c0 = half * kColsPerHalf; c0 < (half + 1) * kColsPerHalf && c0 < BN; c0 += 16) {
        float v[16];
        if (have_acc) {
          tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) my_part[(c0 + j) * kBM + quad * 32 + lane] = v[j];
      }
    }
    // the row scales of this thread's four rows are fetched while the cluster barrier is pending
    const int r4 = (tid & 31) * 4, csub = tid >> 5;  // 8 columns in flight per pass
    float wsc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) wsc[i] = (row0 + r4 + i < p.N) ? __ldg(p.scales + row0 + r4 + i) : 0.f;
    cluster.sync();
    const int rank = (int)cluster.block_rank(), nranks = p.ksplit;
    // this CTA's columns: rank, rank + nranks, ...; 32 threads x float4 cover the 128 rows of a column
    if (tid < kProducerWarps * 32) {
      for (int c = rank + csub * nranks; c < BN; c += kProducerWarps * nranks) {
        const int m = m0 + c, rr = row0 + r4;
        const float as = m < p.M ? __ldg(p.act_scale + m) : 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < nranks; ++r) {
          const float4 v = *reinterpret_cast<const float4*>(cluster.map_shared_rank(my_part, r) + c * kBM + r4);
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (m < p.M && rr < p.N) {
          const float v0 = acc.x * wsc[0] * as;
          const float v1 = acc.y * wsc[1] * as;
          const float v2 = acc.z * wsc[2] * as;
          const float v3 = acc.w * wsc[3] * as;
          if (p.epi == PI_EPI_SWIGLU) {
            float* o = p.out + (size_t)m * p.out_stride + (rr >> 1);
            if (rr + 1 < p.N) o[0] = silu_mul(v0, v1);
            if (rr + 3 < p.N) o[1] = silu_mul(v2, v3);
          } else {
            float* o = p.out + (size_t)m * p.out_stride + rr;
            const bool add = p.epi == PI_EPI_ADD;
            o[0] = add ? o[0] + v0 : v0;
            if (rr + 1 < p.N) o[1] = add ? o[1] + v1 : v1;
            if (rr + 2 < p.N) o[2] = add ? o[2] + v2 : v2;
            if (rr + 3 < p.N) o[3] = add ? o[3] + v3 : v3;
          }
        }
      }
    }
    cluster.sync();  // nobody leaves while a peer may still be reading its tile
  }
  pi_grid_launch_dependents();

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kProducerWarps + 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
}

// ---- the same GEMM with the weight operand in tensor memory ----------------------------------------------------
//
// The kernel above is bound by shared-memory bandwidth, not by HBM: per K block every CTA writes 32 KiB of widened
// weights to shared memory, the two MMAs of a K step each read the 4 KiB weight slice again, and the activation
// planes add as much.  Here the widened weights never touch shared memory: a producer thread owns one weight row
// (= one TMEM lane), loads 64 bytes of it straight from global memory with two 256-bit loads, widens them to 32
// packed fp16 pairs and stores them with one tcgen05.st into the stage's 64 TMEM columns; the MMA takes A from TMEM.
// The hi and lo activation planes are one B tile of 2*BN rows (hi rows, then lo rows), so one MMA per K step reads
// the weights once and leaves W*hi in accumulator columns [0, BN) and W*lo in [BN, 2*BN); the epilogue adds them.
// Shared memory then only carries the activation tiles (TMA in, MMA out).
//
// TMEM columns: [0, 2*BN) accumulator, then STAGES x 64 columns of widened weights.  The kernel always asks for
// all 512 columns and for at least kMinSmem of shared memory, so two of these CTAs (or one of these and one of the
// kernel above) never share an SM: a CTA blocked in tcgen05.alloc while its cluster peers wait for it at a cluster
// barrier could otherwise deadlock.
constexpr int kACols = kBK / 2;           // 128 fp16 of a row = 64 32-bit TMEM columns
constexpr size_t kMinSmem = 120 * 1024;

__device__ __forceinline__ void ld_stream_32(const void* p, uint32_t* v) {
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "l"(p));
}

// 32 consecutive TMEM columns of this thread's lane (lane = 32 * (warp % 4) + laneid).
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}

// D[tmem_d] (+)= A[tmem_a] * B[smem descriptor]
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_ta_kernel(const GemmParams p, const __grid_constant__ CUtensorMap map_act) {
  constexpr int kBAtomBytes = 2 * BN * 128;                 // one 64-element K atom: BN hi rows, then BN lo rows
  constexpr int kBStageBytes = 2 * kBAtomBytes;
  constexpr int kDCols = 2 * BN;
  static_assert(kDCols + STAGES * kACols <= 512, "TMEM holds 512 columns");
  constexpr int kTmemCols = 512;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bars[2 * STAGES + 1];
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = warp & 3, half = (warp >> 2) & 1;
  const int row0 = blockIdx.x * kBM, m0 = blockIdx.z * BN;
  const int kb_begin = (int)((long)blockIdx.y * p.nkb / p.ksplit), kb_end = (int)((long)(blockIdx.y + 1) * p.nkb / p.ksplit);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), accum_bar = smem_u32(&bars[2 * STAGES]);
  // Every thread releases the dependent grid right away (the release only happens once all threads of all CTAs
  // have done so): the next kernels then sit resident, with their own prologue done, by the time this one ends.
  pi_grid_launch_dependents();

  // ---- weight producers (warps 0-7): thread = weight row quad*32+lane, K half `half` of every K block ----------
  // A GROUP of kGroup K blocks (2 x 32 bytes each) is requested one group ahead of the one being widened; the
  // first group goes out before anything else in the kernel (weights never depend on the preceding kernel).
  constexpr int kGroup = 4;
  const unsigned char* src = nullptr;
  uint32_t cur[kGroup][16], nxt[kGroup][16];
  auto load_group = [&](uint32_t (&g)[kGroup][16], int kb0) {
#pragma unroll
    for (int d = 0; d < kGroup; ++d)
      if (kb0 + d < kb_end) {
        ld_stream_32(src + (size_t)(kb0 + d) * kBK, &g[d][0]);
        ld_stream_32(src + (size_t)(kb0 + d) * kBK + 32, &g[d][8]);
      }
  };
  if (warp < kProducerWarps) {
    const int row = min(row0 + quad * 32 + lane, p.N - 1);
    src = reinterpret_cast<const unsigned char*>(p.W) + (size_t)row * p.ld + half * 64;
    load_group(cur, kb_begin);
  }

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, kProducerWarps + 1);       // one arrival per producer warp + the TMA thread's expect_tx
      mbar_init(empty0 + 8 * s, 1);                        // one tcgen05.commit
    }
    mbar_init(accum_bar, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kProducerWarps + 1) {  // TMEM allocation is warp-wide
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;
  const uint32_t tmem_a0 = tmem + (uint32_t)kDCols;
  const uint32_t smem_base = smem_u32(smem);

  if (warp < kProducerWarps) {
    bool stop = false;
    const uint32_t my_a = tmem_a0 + ((uint32_t)(quad * 32) << 16) + (uint32_t)(half * 32);
    for (int kb0 = kb_begin; kb0 < kb_end && !stop; kb0 += kGroup) {
      if (kb0 + kGroup < kb_end) load_group(nxt, kb0 + kGroup);
#pragma unroll
      for (int d = 0; d < kGroup; ++d) {
        const int kb = kb0 + d;
        if (kb >= kb_end || stop) break;
        const int it = kb - kb_begin, s = it % STAGES;
        uint32_t h[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) widen4(cur[d][i], h[2 * i], h[2 * i + 1]);
        // lane 0 polls for the whole warp
        int ok = 1;
        if (lane == 0) ok = (!s_abort && mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1)) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0 && !s_abort) {
            s_abort = 1;
            if (p.err_flag) atomicExch(p.err_flag, 2);
          }
          stop = true;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");   // the MMAs that read this stage are done
        tmem_st32(my_a + (uint32_t)(s * kACols), h);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * s);
      }
#pragma unroll
      for (int d = 0; d < kGroup; ++d)
#pragma unroll
        for (int i = 0; i < 16; ++i) cur[d][i] = nxt[d][i];
    }
    pi_grid_dependency_wait();  // the epilogue below touches memory the producer kernel may still be writing
  } else if (warp == kProducerWarps) {
    // ---- activation loader: one 3-D TMA box {64 K, BN rows, 2 planes} per K atom -------------------------------
    if (lane == 0) {
      pi_grid_dependency_wait();  // the activation planes come from the preceding kernel
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int it = kb - kb_begin, s = it % STAGES;
        if (s_abort) break;
        if (!mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1)) {
          s_abort = 1;
          if (p.err_flag) atomicExch(p.err_flag, 3);
          break;
        }
        const uint32_t bar = full0 + 8 * s;
        const uint32_t b_stage = smem_base + s * kBStageBytes;
        mbar_arrive_expect_tx(bar, kBStageBytes);
#pragma unroll
        for (int atom = 0; atom < 2; ++atom) {
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
                  b_stage + atom * kBAtomBytes),
              "l"(&map_act), "r"(bar), "r"(kb * kBK + atom * 64), "r"(m0), "r"(0)
              : "memory");
        }
      }
    }
  } else {
    // ---- MMA issuer ------------------------------------------------------------------------------------------
    if (lane == 0) {
      // kind::f16, D = f32, A (TMEM) and B (shared, K-major) = f16, N = 2*BN, M = 128
      const uint32_t idesc = (1u << 4) | ((uint32_t)(kDCols >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int it = kb - kb_begin, s = it % STAGES;
        if (s_abort || !mbar_wait(full0 + 8 * s, (it / STAGES) & 1)) {
          if (!s_abort && p.err_flag) atomicExch(p.err_flag, 4);
          s_abort = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t db0 = smem_desc(smem_base + s * kBStageBytes);
        const uint32_t a_s = tmem_a0 + (uint32_t)(s * kACols);
#pragma unroll
        for (int atom = 0; atom < 2; ++atom) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {  // 16 K elements: 8 TMEM columns of A, 32 bytes of every B row
            const uint64_t db = db0 + (uint64_t)((atom * kBAtomBytes + ks * 32) >> 4);
            umma_f16_ts(tmem, a_s + (uint32_t)((atom * 4 + ks) * 8), db, idesc, (kb > kb_begin || atom + ks > 0) ? 1u : 0u);
          }
        }
        umma_commit(empty0 + 8 * s);  // the stage (TMEM columns and shared tile) is free once these MMAs are done
      }
      if (ok) umma_commit(accum_bar);
    }
  }

  // ---- epilogue: warp w owns TMEM lanes 32*(w%4).., the two column halves go to warps 0-3 / 4-7 -----------------
  bool have_acc = false;
  if (warp < kProducerWarps) {
    int got = 0;
    if (lane == 0) {
      got = ((kb_begin < kb_end) && !s_abort && mbar_wait(accum_bar, 0)) ? 1 : 0;
      if (kb_begin < kb_end && !got && !s_abort) {
        s_abort = 1;
        if (p.err_flag) atomicExch(p.err_flag, 5);
      }
    }
    have_acc = __shfl_sync(0xffffffffu, got, 0) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  const int row = row0 + quad * 32 + lane;
  constexpr int kColsPerHalf = BN / 2 >= 16 ? BN / 2 : 16;  // BN 16: only the first half works
  const bool epi_warp = warp < kProducerWarps && (BN >= 32 || half == 0);
  const uint32_t my_d = tmem + ((uint32_t)(quad * 32) << 16);

  if (p.ksplit == 1) {
    if (epi_warp && have_acc) {
      const float ws = row < p.N ? p.scales[row] : 0.f;
#pragma unroll 1
      for (int c0 = half * kColsPerHalf; c0 < (half + 1) * kColsPerHalf && c0 < BN; c0 += 16) {
        float v[16], w[16];
        tmem_ld16(my_d + (uint32_t)c0, v);
        tmem_ld16(my_d + (uint32_t)(BN + c0), w);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + c0 + j;
          const float as = m < p.M ? p.act_scale[m] : 0.f;
          emit(p, m, row, (v[j] + w[j]) * ws * as, lane);
        }
      }
    }
  } else {
    // K split over the CTAs of a cluster: same rank-ordered reduction through distributed shared memory as above.
    cg::cluster_group cluster = cg::this_cluster();
    float* my_part = reinterpret_cast<float*>(smem);  // [BN][128]
    if (epi_warp) {
#pragma unroll 1
      for (int c0 = half * kColsPerHalf; c0 < (half + 1) * kColsPerHalf && c0 < BN; c0 += 16) {
        float v[16], w[16];
        if (have_acc) {
          tmem_ld16(my_d + (uint32_t)c0, v);
          tmem_ld16(my_d + (uint32_t)(BN + c0), w);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = w[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) my_part[(c0 + j) * kBM + quad * 32 + lane] = v[j] + w[j];
      }
    }
    const int r4 = (tid & 31) * 4, csub = tid >> 5;  // 8 columns in flight per pass
    float wsc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) wsc[i] = (row0 + r4 + i < p.N) ? __ldg(p.scales + row0 + r4 + i) : 0.f;
    cluster.sync();
    const int rank = (int)cluster.block_rank(), nranks = p.ksplit;
    if (tid < kProducerWarps * 32) {
      for (int c = rank + csub * nranks; c < BN; c += kProducerWarps * nranks) {
        const int m = m0 + c, rr = row0 + r4;
        const float as = m < p.M ? __ldg(p.act_scale + m) : 0.f;
        // all peers' slices are requested before the first add (one remote latency instead of nranks), the adds
        // stay in rank order
        float4 part[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          part[r] = r < nranks ? *reinterpret_cast<const float4*>(cluster.map_shared_rank(my_part, r) + c * kBM + r4)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          acc.x += part[r].x; acc.y += part[r].y; acc.z += part[r].z; acc.w += part[r].w;
        }
        if (m < p.M && rr < p.N) {
          const float v0 = acc.x * wsc[0] * as;
          const float v1 = acc.y * wsc[1] * as;
          const float v2 = acc.z * wsc[2] * as;
          const float v3 = acc.w * wsc[3] * as;
          if (p.epi == PI_EPI_SWIGLU) {
            float* o = p.out + (size_t)m * p.out_stride + (rr >> 1);
            if (rr + 1 < p.N) o[0] = silu_mul(v0, v1);
            if (rr + 3 < p.N) o[1] = silu_mul(v2, v3);
          } else {
            float* o = p.out + (size_t)m * p.out_stride + rr;
            const bool add = p.epi == PI_EPI_ADD;
            o[0] = add ? o[0] + v0 : v0;
            if (rr + 1 < p.N) o[1] = add ? o[1] + v1 : v1;
            if (rr + 2 < p.N) o[2] = add ? o[2] + v2 : v2;
            if (rr + 3 < p.N) o[3] = add ? o[3] + v3 : v3;
          }
        }
      }
    }
    cluster.sync();  // nobody leaves while a peer may still be reading its tile
  }
  pi_grid_launch_dependents();

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kProducerWarps + 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
}

// ---- activation preparation: optional RMSNorm, power-of-two row scaling, fp16 hi/lo split ---------------------
// Register-resident version: one CTA per activation row, the row is read from global memory exactly once
// (VPT float4 per thread), two block reductions (sum of squares, then max |y|), one vectorised write per plane.
template <int VPT>
__global__ void __launch_bounds__(256) act_split_reg_kernel(const float* __restrict__ x, size_t x_stride,
                                                            const float* __restrict__ norm_weight, float eps, int K,
                                                            __half* __restrict__ hi, __half* __restrict__ lo,
                                                            float* __restrict__ act_scale) {
  __shared__ float red[8];
  __shared__ float s_val;
  pi_grid_dependency_wait();
  const int m = blockIdx.x, tid = threadIdx.x, n4 = K >> 2;
  const float4* row = reinterpret_cast<const float4*>(x + (size_t)m * x_stride);
  float4 v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = tid + i * 256;
    v[i] = idx < n4 ? row[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (norm_weight) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
    ss = pi_warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) t += red[i];
      s_val = 1.0f / sqrtf(t / (float)K + eps);
    }
    __syncthreads();
    const float inv = s_val;
    const float4* nw = reinterpret_cast<const float4*>(norm_weight);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * 256;
      if (idx < n4) {
        const float4 w = __ldg(nw + idx);
        v[i].x = v[i].x * inv * w.x;
        v[i].y = v[i].y * inv * w.y;
        v[i].z = v[i].z * inv * w.z;
        v[i].w = v[i].w * inv * w.w;
      }
    }
    __syncthreads();  // red[] and s_val are reused below
  }
  float mx = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
  mx = pi_warp_max(mx);
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t = fmaxf(t, red[i]);
    int e = 0;
    if (t > 0.f && t < INFINITY) frexpf(t, &e);
    s_val = ldexpf(1.0f, -e);
    act_scale[m] = ldexpf(1.0f, e);
  }
  __syncthreads();
  const float s = s_val;
  uint2* hrow = reinterpret_cast<uint2*>(hi + (size_t)m * K);
  uint2* lrow = reinterpret_cast<uint2*>(lo + (size_t)m * K);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = tid + i * 256;
    if (idx < n4) {
      const float y[4] = {v[i].x * s, v[i].y * s, v[i].z * s, v[i].w * s};
      __half h[4], l[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        h[j] = __float2half_rn(y[j]);
        l[j] = __float2half_rn(y[j] - __half2float(h[j]));
      }
      hrow[idx] = make_uint2((uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16),
                             (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16));
      lrow[idx] = make_uint2((uint32_t)__half_as_ushort(l[0]) | ((uint32_t)__half_as_ushort(l[1]) << 16),
                             (uint32_t)__half_as_ushort(l[2]) | ((uint32_t)__half_as_ushort(l[3]) << 16));
    }
  }
}

// General version (any K): the normalised row is parked in shared memory between the passes.
__global__ void __launch_bounds__(256) act_split_kernel(const float* __restrict__ x, size_t x_stride,
                                                        const float* __restrict__ norm_weight, float eps, int K,
                                                        __half* __restrict__ hi, __half* __restrict__ lo,
                                                        float* __restrict__ act_scale) {
  extern __shared__ float ys[];
  __shared__ float red[8];
  __shared__ float s_val;
  pi_grid_dependency_wait();
  const int m = blockIdx.x, tid = threadIdx.x;
  const float* row = x + (size_t)m * x_stride;
  float inv = 1.0f;
  if (norm_weight) {
    float ss = 0.f;
    for (int k = tid; k < K; k += blockDim.x) ss = fmaf(row[k], row[k], ss);
    ss = pi_warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
      s_val = 1.0f / sqrtf(t / (float)K + eps);
    }
    __syncthreads();
    inv = s_val;
    __syncthreads();
  }
  float mx = 0.f;
  for (int k = tid; k < K; k += blockDim.x) {
    const float y = norm_weight ? row[k] * inv * norm_weight[k] : row[k];
    ys[k] = y;
    mx = fmaxf(mx, fabsf(y));
  }
  mx = pi_warp_max(mx);
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t = fmaxf(t, red[i]);
    int e = 0;
    if (t > 0.f && t < INFINITY) frexpf(t, &e);   // t = f * 2^e, f in [0.5, 1)
    s_val = ldexpf(1.0f, -e);                     // scaled row max lands in [0.5, 1)
    act_scale[m] = ldexpf(1.0f, e);
  }
  __syncthreads();
  const float s = s_val;
  for (int k = tid; k < K; k += blockDim.x) {
    const float y = ys[k] * s;                    // exact: power-of-two scaling
    const __half h = __float2half_rn(y);
    hi[(size_t)m * K + k] = h;
    lo[(size_t)m * K + k] = __float2half_rn(y - __half2float(h));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

int pick_bn(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128; }

template <int BN, int STAGES>
cudaError_t launch_tc(pi_ctx* ctx, const GemmParams& p, const CUtensorMap& hi, const CUtensorMap& lo, dim3 grid) {
  constexpr size_t smem = (size_t)STAGES * (kATileBytes + 4 * BN * 128) + 1024;
  auto k = gemm_tc_kernel<BN, STAGES>;
  static bool granted = false;  // per instantiation
  if (!granted) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    granted = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (ctx->opt_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (grid.y > 1) {  // the K slices of one row tile form a cluster
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = grid.y;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, k, p, hi, lo);
}

template <int BN, int STAGES>
cudaError_t launch_ta(pi_ctx* ctx, const GemmParams& p, const CUtensorMap& act, dim3 grid) {
  constexpr size_t smem = std::max((size_t)STAGES * (4 * BN * 128) + 1024, kMinSmem);
  auto k = gemm_ta_kernel<BN, STAGES>;
  static bool granted = false;  // per instantiation
  if (!granted) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    granted = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (ctx->opt_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (grid.y > 1) {  // the K slices of one row tile form a cluster
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = grid.y;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, k, p, act);
}

}  // namespace

bool pi_gemm_tc_supported(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a) {
  (void)ctx;
  if (lin->kind != PI_INT8) return false;
  if (lin->cols % kBK != 0 || lin->ld != lin->cols) return false;   // whole K blocks, 16-byte aligned rows
  if (lin->rows < 32) return false;
  if (a.epi == PI_EPI_SWIGLU && (lin->rows % 2) != 0) return false;
  if (lin->cols > 65536 * 2) return false;
  return encode_tiled() != nullptr;
}

pi_status pi_launch_gemm_tc(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a) {
  PI_REQUIRE(ctx, pi_gemm_tc_supported(ctx, lin, a), "tensor-core GEMM does not support this projection");
  const int M = a.M, K = (int)lin->cols, N = (int)lin->rows;
  const int BN = pick_bn(M);
  const int mtiles = (M + BN - 1) / BN, M_pad = mtiles * BN;
  const int rtiles = (N + kBM - 1) / kBM;
  const int nkb = K / kBK;

  // K splits: as many as still fit in ONE wave (a CTA owns its SM, so a second, partly filled wave would cost a
  // whole extra prologue + epilogue), at least two K blocks each.
  int ksplit = 1;
  const int tiles = rtiles * mtiles;
  if (tiles < ctx->sm_count) {
    const int want = std::min(std::max(1, ctx->sm_count / tiles), std::max(1, nkb / 2));
    while (ksplit * 2 <= want && ksplit < 8) ksplit *= 2;   // a portable cluster holds up to 8 CTAs
  }

  // scratch (global memory beyond the inputs and outputs): [act hi | act lo | act_scale]
  const size_t plane = (size_t)M_pad * K * sizeof(__half);
  PI_TRY(pi_reserve(ctx, &ctx->gemm_act, 2 * plane + (size_t)M_pad * sizeof(float) + 256));
  __half* hi = static_cast<__half*>(ctx->gemm_act.ptr);
  __half* lo = hi + (size_t)M_pad * K;
  float* act_scale = reinterpret_cast<float*>(lo + (size_t)M_pad * K);

  pi_prof_scope prof(ctx, PI_PROF_GEMM_TC);
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = (size_t)K * sizeof(float);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
    static size_t split_granted = 48 * 1024;
    if (cfg.dynamicSmemBytes > split_granted) {
      PI_CUDA(ctx, cudaFuncSetAttribute(act_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cfg.dynamicSmemBytes));
      split_granted = cfg.dynamicSmemBytes;
    }
    cudaError_t e;
    const int n4 = K / 4;
    const bool vec_ok = ((uintptr_t)a.x % 16 == 0) && (a.x_stride % 4 == 0) &&
                        (!a.norm_weight || (uintptr_t)a.norm_weight % 16 == 0) && n4 <= 256 * 16;
    if (vec_ok) {  // the row fits the registers of one CTA: single pass
      cfg.dynamicSmemBytes = 0;
      if (n4 <= 256 * 2) e = cudaLaunchKernelEx(&cfg, act_split_reg_kernel<2>, a.x, a.x_stride, a.norm_weight, a.norm_eps, K, hi, lo, act_scale);
      else if (n4 <= 256 * 4) e = cudaLaunchKernelEx(&cfg, act_split_reg_kernel<4>, a.x, a.x_stride, a.norm_weight, a.norm_eps, K, hi, lo, act_scale);
      else if (n4 <= 256 * 8) e = cudaLaunchKernelEx(&cfg, act_split_reg_kernel<8>, a.x, a.x_stride, a.norm_weight, a.norm_eps, K, hi, lo, act_scale);
      else e = cudaLaunchKernelEx(&cfg, act_split_reg_kernel<16>, a.x, a.x_stride, a.norm_weight, a.norm_eps, K, hi, lo, act_scale);
    } else {
      e = cudaLaunchKernelEx(&cfg, act_split_kernel, a.x, a.x_stride, a.norm_weight, a.norm_eps, K, hi, lo, act_scale);
    }
    if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "activation split launch failed: %s", cudaGetErrorString(e));
    ctx->launches++;
  }

  const bool a_in_tmem = ctx->opt_gemm_a_tmem && ((uintptr_t)lin->w % 32 == 0) && (lin->ld % 32 == 0);
  CUtensorMap maps[2];
  if (a_in_tmem) {
    // one map over both planes: {K, M rows (rows past M read as zero), 2 planes M_pad*K apart}
    const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, 2};
    const cuuint64_t strides[2] = {(cuuint64_t)K * sizeof(__half), (cuuint64_t)M_pad * K * sizeof(__half)};
    const cuuint32_t box[3] = {64, (cuuint32_t)BN, 2};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_tiled()(&maps[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, (void*)hi, dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return pi_fail(ctx, PI_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  } else {
    for (int i = 0; i < 2; ++i) {
      const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};          // innermost first; rows past M read as zero
      const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(__half)};
      const cuuint32_t box[2] = {64, (cuuint32_t)BN};
      const cuuint32_t estr[2] = {1, 1};
      CUresult r = encode_tiled()(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, i == 0 ? (void*)hi : (void*)lo, dims, strides, box,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return pi_fail(ctx, PI_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    }
  }

  GemmParams p;
  p.W = static_cast<const int8_t*>(lin->w);
  p.scales = lin->scales;
  p.act_scale = act_scale;
  p.out = a.out;
  p.ld = lin->ld;
  p.out_stride = a.out_stride;
  p.N = N;
  p.K = K;
  p.M = M;
  p.ksplit = ksplit;
  p.nkb = nkb;
  p.epi = a.epi;
  p.err_flag = ctx->dev_err;
  const dim3 grid(rtiles, ksplit, mtiles);
  cudaError_t e;
  if (a_in_tmem) {
    switch (BN) {
      case 16: e = launch_ta<16, 6>(ctx, p, maps[0], grid); break;
      case 32: e = launch_ta<32, 6>(ctx, p, maps[0], grid); break;
      case 64: e = launch_ta<64, 6>(ctx, p, maps[0], grid); break;
      default: e = launch_ta<128, 3>(ctx, p, maps[0], grid); break;
    }
  } else {
    switch (BN) {
      case 16: e = launch_tc<16, 4>(ctx, p, maps[0], maps[1], grid); break;
      case 32: e = launch_tc<32, 4>(ctx, p, maps[0], maps[1], grid); break;
      case 64: e = launch_tc<64, 3>(ctx, p, maps[0], maps[1], grid); break;
      default: e = launch_tc<128, 2>(ctx, p, maps[0], maps[1], grid); break;
    }
  }
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "tensor-core GEMM launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  return PI_OK;
}

// ---- pi_linear_apply_noalloc -----------------------------------------------------------------------------------
//
// The tensor-core projection needs scratch in global memory: the two fp16 planes (hi, lo) the f32 activations are
// split into, plus one power-of-two factor per activation row.  pi_linear_apply takes that scratch from a buffer the
// context grows with cudaMalloc on demand.  Some callers must not allocate at the moment they run a projection:
// a serving loop that is inside a CUDA stream capture (cudaMalloc is not a capturable operation and invalidates
// the capture), a host thread with a latency budget that a driver allocation (which can take the device-wide
// allocation lock and synchronise) would break, or an embedder that has handed all device memory to its own pool.
// For them the same kernels run here against a fixed scratch area that is part of the library image: every GPU
// that loads the library carries kNoAllocScratchBytes (about 2 MiB) of it until the process exits.
//
// Limits: int8 projections the tensor path supports (columns a multiple of 128), 1 <= M <= 64 activation rows,
// columns <= 8192.  Larger shapes are refused with PI_ERR_INVALID_ARG; they are never silently routed elsewhere.
//
// The area is shared by every call on the device and keeps whatever the previous call left in it.  Nothing in it
// has to start at zero: rows [0, M) of both planes and the M factors are rewritten by every call before they are
// read, and rows >= M are never read (the TMA descriptor is M rows tall, so a box that reaches past row M is
// zero-filled by the copy engine rather than fetched).  Two calls whose kernels overlap on the GPU - different
// streams, or different contexts on one device - would overwrite each other's planes: callers must order them.
//
// Set-up happens inside the first call on each device: the address of the area is looked up with
// cudaGetSymbolAddress and, the first time each tile width is used, the kernel's shared-memory limit is raised
// with cudaFuncSetAttribute.  Neither allocates, but make that first call before any stream capture begins.
// The call itself never calls cudaMalloc, cudaFree, or any allocating library routine.
constexpr int kNoAllocMaxM = 64;
constexpr int kNoAllocMaxK = 8192;
constexpr size_t kNoAllocScratchBytes =
    2 * (size_t)kNoAllocMaxM * kNoAllocMaxK * sizeof(__half) + (size_t)kNoAllocMaxM * sizeof(float) + 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not an address a kernel could use.  Its device
// address is looked up once per device, with that device current, and cached here.
static void* g_noalloc_addr[64] = {};

static pi_status noalloc_scratch_address(pi_ctx* ctx, void** out) {
  PI_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, "device index %d is outside the table of scratch addresses", ctx->device);
  if (!g_noalloc_addr[ctx->device]) {
    int current = -1;
    PI_CUDA(ctx, cudaGetDevice(&current));
    if (current != ctx->device) PI_CUDA(ctx, cudaSetDevice(ctx->device));
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (current != ctx->device) cudaSetDevice(current);
    if (e != cudaSuccess || !ptr)
      return pi_fail(ctx, PI_ERR_CUDA, "cudaGetSymbolAddress for the built-in scratch failed: %s", cudaGetErrorString(e));
    g_noalloc_addr[ctx->device] = ptr;
  }
  *out = g_noalloc_addr[ctx->device];
  return PI_OK;
}

extern "C" pi_status pi_linear_apply_noalloc(pi_ctx* ctx, const pi_linear* lin, const float* x_dev, float* out_dev, int M) {
  if (!ctx) return PI_ERR_INVALID_ARG;
  PI_REQUIRE(ctx, lin && x_dev && out_dev, "null pointer");
  PI_REQUIRE(ctx, M >= 1 && M <= kNoAllocMaxM, "batch %d is outside the built-in scratch (1..%d activation rows)", M, kNoAllocMaxM);
  PI_REQUIRE(ctx, lin->cols <= (size_t)kNoAllocMaxK, "%zu columns exceed the built-in scratch (at most %d)", lin->cols, kNoAllocMaxK);
  pi_linear_args a;
  a.x = x_dev;
  a.x_stride = lin->cols;
  a.out = out_dev;
  a.out_stride = lin->rows;
  a.M = M;
  PI_REQUIRE(ctx, pi_gemm_tc_supported(ctx, lin, a),
             "the allocation-free projection needs an int8 matrix with at least 32 rows and a multiple of 128 columns");
  void* scratch = nullptr;
  PI_TRY(noalloc_scratch_address(ctx, &scratch));

  const int K = (int)lin->cols, N = (int)lin->rows;
  const int BN = pick_bn(M);
  const int mtiles = 1, M_pad = BN;
  const int rtiles = (N + kBM - 1) / kBM;
  const int nkb = K / kBK;
  int ksplit = 1;
  if (rtiles < ctx->sm_count) {
    const int want = std::min(std::max(1, (ctx->sm_count * 3 / 2) / rtiles), std::max(1, nkb / 2));
    while (ksplit * 2 <= want && ksplit < 8) ksplit *= 2;
  }
  __half* hi = static_cast<__half*>(scratch);
  __half* lo = hi + (size_t)M_pad * K;
  float* act_scale = reinterpret_cast<float*>(lo + (size_t)M_pad * K);

  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = (size_t)K * sizeof(float);  // at most 32 KiB here: no attribute change needed
    cfg.stream = ctx->stream;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, act_split_kernel, x_dev, (size_t)K, (const float*)nullptr, 0.f, K, hi, lo, act_scale);
    if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "activation split launch failed: %s", cudaGetErrorString(e));
    ctx->launches++;
  }
  CUtensorMap maps[2];
  for (int i = 0; i < 2; ++i) {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(__half)};
    const cuuint32_t box[2] = {64, (cuuint32_t)BN};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_tiled()(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, i == 0 ? (void*)hi : (void*)lo, dims, strides,
                                      box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return pi_fail(ctx, PI_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  }
  GemmParams p;
  p.W = static_cast<const int8_t*>(lin->w);
  p.scales = lin->scales;
  p.act_scale = act_scale;
  p.out = out_dev;
  p.ld = lin->ld;
  p.out_stride = lin->rows;
  p.N = N;
  p.K = K;
  p.M = M;
  p.ksplit = ksplit;
  p.nkb = nkb;
  p.epi = PI_EPI_STORE;
  p.err_flag = ctx->dev_err;
  const dim3 grid(rtiles, ksplit, mtiles);
  cudaError_t e;
  switch (BN) {
    case 16: e = launch_tc<16, 4>(ctx, p, maps[0], maps[1], grid); break;
    case 32: e = launch_tc<32, 4>(ctx, p, maps[0], maps[1], grid); break;
    default: e = launch_tc<64, 3>(ctx, p, maps[0], maps[1], grid); break;
  }
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "tensor-core GEMM launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  return PI_OK;
}
