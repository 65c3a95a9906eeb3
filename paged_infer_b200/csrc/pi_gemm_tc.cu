// Tensor-core dequant GEMM for batched decode and prefill: tcgen05.mma with the
// accumulator AND the weight operand in tensor memory (TMEM), for int8 weights and
// f32 activations.
//
//   out[m][r] = scale[r] * row_factor[m] * sum_k W[r][k] * y[m][k]
//
// Swap-AB: the 128 weight rows of a CTA sit on the MMA's M axis, the batch on its N
// axis.  A producer thread owns one weight row (= one TMEM lane): it loads 32 bytes
// of the row with one 256-bit load, widens the int8 codes to bf16 (exact) in
// registers and stores the 16 packed pairs with one tcgen05.st into the stage's 64
// TMEM columns (four threads, in four warps, share a row's K block); the MMA takes A from TMEM, so widened weights never touch shared
// memory.  Each f32 activation y is carried as three bf16 planes whose sum is y
// exactly (p0 = bf16(y), p1 = bf16(y - p0), p2 = bf16(y - p0 - p1)); the three
// planes of a K atom are ONE B tile of 3*BN rows fetched by one 3-D TMA box
// (cp.async.bulk.tensor, CTA-local), so one MMA per K step reads the weights
// once and leaves W*p0, W*p1, W*p2 in three groups of accumulator columns, which
// the epilogue adds.  Every product int8 x bf16 is exact and accumulation is f32:
// the result is f32-equivalent whatever the magnitude of a row.
//
// The planes come either from the activation-split kernel below (optionally with
// RMSNorm: planes of x * norm_weight, row factor 1/rms) or straight from the epilogue
// of the projection that produced the activation (`emit`): that epilogue writes its
// f32 result and, in the same pass, the three planes of result * next_norm_weight
// and per-tile partial sums of result^2, from which the consumer derives 1/rms.
//
// Warp roles (18 warps): 0-15 stream + widen the weights and later run the epilogue
// (0-7 read the accumulator out of TMEM); warp 16 issues the TMA loads of the
// activations; warp 17 allocates TMEM and issues the MMAs.  Stages are handed over with mbarriers; every wait is
// bounded and a wait that runs out raises the context's error word instead of
// hanging.
//
// K is split across CTAs when there are too few row tiles to fill the SMs; the K
// slices of one row tile form a thread-block cluster and add their partial tiles
// through distributed shared memory in rank order, so results do not depend on
// timing.
//
// Replaces math::matmat_i8_weight_parallel + transpose_rb_to_br for batches beyond a
// few rows (reference src/math.rs:223-290), with math::rms_norm (src/math.rs:4-22)
// folded in.
#include <cooperative_groups.h>
#include <cuda.h>
#include <stdlib.h>

#include <algorithm>

#include "pi_common.cuh"

namespace cg = cooperative_groups;

#include "pi_gemm_tc.cuh"

namespace {
using namespace pi_tc;

// PUSH (launches whose K is split over a cluster): the partial tiles meet by remote stores into a receive area of the
// CTA that owns the column, behind the pipeline stages, instead of by remote loads from every CTA's parked tile.
template <int BN, int STAGES, bool PUSH>
__global__ void __launch_bounds__(kThreads, 1)
gemm_ta_kernel(const GemmParams p, const __grid_constant__ CUtensorMap map_act) {
  constexpr int kBAtomBytes = kPlanes * BN * 128;           // one 64-element K atom: BN rows of plane 0, 1, 2
  constexpr int kBStageBytes = 2 * kBAtomBytes;
  constexpr int kDCols = kPlanes * BN;
  constexpr int kAStart = (kDCols + 63) / 64 * 64;          // weight stages start on a 64-column boundary
  static_assert(kDCols <= 256, "one MMA covers at most 256 accumulator columns");
  static_assert(kAStart + STAGES * kACols <= 512, "TMEM holds 512 columns");
  constexpr int kTmemCols = 512;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bars[2 * STAGES + 1];
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_abort;
  __shared__ volatile int s_dep_ok;   // the preceding kernel has completed: from here on waits are this kernel's own
  __shared__ float s_rowf[BN];     // row factor of the activation rows of this CTA

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = warp & 3, kq = (warp >> 2) & 3, half = (warp >> 2) & 1;
  const int row0 = blockIdx.x * kBM, m0 = blockIdx.z * BN;
  const int kb_begin = (int)((long)blockIdx.y * p.nkb / p.ksplit), kb_end = (int)((long)(blockIdx.y + 1) * p.nkb / p.ksplit);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), accum_bar = smem_u32(&bars[2 * STAGES]);

  // ---- weight producers (warps 0-15): thread = weight row quad*32+lane, K quarter `kq` of every K block --------
  // A GROUP of kGroup K blocks (32 bytes each) is requested one group ahead of the one being widened; the first
  // group goes out before anything else in the kernel (weights never depend on the preceding kernel).
  constexpr int kGroup = 4;
  const unsigned char* src = nullptr;
  uint32_t cur[kGroup][8], nxt[kGroup][8];
  auto load_group = [&](uint32_t (&g)[kGroup][8], int kb0) {
#pragma unroll
    for (int d = 0; d < kGroup; ++d)
      if (kb0 + d < kb_end) ld_stream_32(src + (size_t)(kb0 + d) * kBK, &g[d][0]);
  };
  if (warp < kProducerWarps) {
    const int row = min(row0 + quad * 32 + lane, p.N - 1);
    src = reinterpret_cast<const unsigned char*>(p.W) + (size_t)row * p.ld + kq * 32;
    load_group(cur, kb_begin);
  }

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, kProducerWarps + 1);       // one arrival per producer warp + the TMA thread's expect_tx
      mbar_init(empty0 + 8 * s, 1);                        // one tcgen05.commit
    }
    mbar_init(accum_bar, 1);
    s_abort = 0;
    s_dep_ok = 0;
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
  // A CTA's shared memory may only be written by its cluster peers once it runs: everybody says so now and checks,
  // for free, right before the first remote store of the epilogue.
  if (PUSH) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  // Every thread releases the dependent grid (the release only happens once all threads of all CTAs have done so):
  // the next kernels then sit resident, with their own prologue done, by the time this one ends.  Only now that this
  // CTA holds its tensor memory: a dependent CTA that took the SM's columns first would keep them until this grid
  // completes, and this CTA would wait for them for ever.
  pi_grid_launch_dependents();
  const uint32_t tmem = s_tmem;
  const uint32_t tmem_a0 = tmem + (uint32_t)kAStart;
  const uint32_t smem_base = smem_u32(smem);

  if (warp < kProducerWarps) {
    bool stop = false;
    const uint32_t my_a = tmem_a0 + ((uint32_t)(quad * 32) << 16) + (uint32_t)(kq * 16);
    for (int kb0 = kb_begin; kb0 < kb_end && !stop; kb0 += kGroup) {
      if (kb0 + kGroup < kb_end) load_group(nxt, kb0 + kGroup);
#pragma unroll
      for (int d = 0; d < kGroup; ++d) {
        const int kb = kb0 + d;
        if (kb >= kb_end || stop) break;
        const int it = kb - kb_begin, s = it % STAGES;
        uint32_t h[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) widen4(cur[d][i], h[2 * i], h[2 * i + 1]);
        // lane 0 polls for the whole warp
        int ok = 1;
        if (lane == 0) ok = (!s_abort && mbar_wait_dep(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, &s_dep_ok)) ? 1 : 0;
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
        tmem_st16(my_a + (uint32_t)(s * kACols), h);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * s);
      }
#pragma unroll
      for (int d = 0; d < kGroup; ++d)
#pragma unroll
        for (int i = 0; i < 8; ++i) cur[d][i] = nxt[d][i];
    }
    pi_grid_dependency_wait();  // the epilogue below touches memory the producer kernel may still be writing
    // row factors of this CTA's activation rows (1/rms from the partial sums of squares, in tile order)
    if (tid < BN) s_rowf[tid] = act_row_factor(p, m0 + tid);
    asm volatile("bar.sync 1, %0;" ::"n"(kProducerWarps * 32) : "memory");
  } else if (warp == kProducerWarps) {
    // ---- activation loader: one 3-D TMA box {64 K, BN rows, 3 planes} per K atom -------------------------------
    if (lane == 0) {
      pi_grid_dependency_wait();  // the activation planes come from the preceding kernel
      s_dep_ok = 1;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int it = kb - kb_begin, s = it % STAGES;
        if (s_abort) break;
        if (!mbar_wait_dep(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, &s_dep_ok)) {
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
      // kind::f16, D = f32, A (TMEM) and B (shared, K-major) = bf16, N = 3*BN, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kDCols >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int it = kb - kb_begin, s = it % STAGES;
        if (s_abort || !mbar_wait_dep(full0 + 8 * s, (it / STAGES) & 1, &s_dep_ok)) {
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
  if (warp < kParkWarps) {
    int got = 0;
    if (lane == 0) {
      got = ((kb_begin < kb_end) && !s_abort && mbar_wait_dep(accum_bar, 0, &s_dep_ok)) ? 1 : 0;
      if (kb_begin < kb_end && !got && !s_abort) {
        s_abort = 1;
        if (p.err_flag) atomicExch(p.err_flag, 5);
      }
    }
    have_acc = __shfl_sync(0xffffffffu, got, 0) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  constexpr int kColsPerHalf = BN / 2 >= 16 ? BN / 2 : 16;  // BN 16: only the first half works
  const bool epi_warp = warp < kParkWarps && (BN >= 32 || half == 0);
  const uint32_t my_d = tmem + ((uint32_t)(quad * 32) << 16);

  {
    // The raw partial tile goes from tensor memory through shared memory: the detour turns the row-per-lane accumulator
    // layout into four adjacent output columns per thread, so every store below is 8 or 16 bytes wide.  When K was
    // split over the CTAs of a thread-block cluster (cluster rank = K slice), column c of the tile is finished by
    // rank c % ksplit: every rank stores its values of that column straight into the owner's receive area
    // (distributed shared memory), one cluster barrier later the owner adds the slices in rank order.
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = PUSH ? (int)cluster.block_rank() : 0, nranks = PUSH ? p.ksplit : 1;
    const int cpo = (BN + nranks - 1) / nranks;                // columns an owner receives from each rank
    float* my_part = reinterpret_cast<float*>(smem);          // !PUSH: [BN][128] over the (free) pipeline stages
    float* recv = reinterpret_cast<float*>(smem + STAGES * kBStageBytes);   // PUSH: [nranks][cpo][128]
    if (PUSH) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // every peer runs (arrived long ago)
    if (epi_warp) {
#pragma unroll 1
      for (int c0 = half * kColsPerHalf; c0 < (half + 1) * kColsPerHalf && c0 < BN; c0 += 16) {
        float v[16];
        if (have_acc) {
          tmem_ld_sum16<BN>(my_d, c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
        if (PUSH) {
          // column c belongs to rank c % nranks, as its column c / nranks; this rank's values go to slice `rank` there
          int owner = c0 % nranks, idx = c0 / nranks;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float* dst = cluster.map_shared_rank(recv, owner) + ((size_t)(rank * cpo + idx) * kBM + quad * 32 + lane);
            *dst = v[j];
            if (++owner == nranks) {
              owner = 0;
              ++idx;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) my_part[(c0 + j) * kBM + quad * 32 + lane] = v[j];
        }
      }
    }
    // this thread's four rows: scales and emit norm weights are fetched while the barrier is pending
    const int r4 = (tid & 31) * 4, csub = tid >> 5;  // 16 columns in flight per pass
    EpiRows rows;
    epi_rows_load(p, row0, tid, rows);
    if (PUSH) {
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // all partials of this CTA's columns are here
    } else {
      __syncthreads();
    }
    if (tid < kProducerWarps * 32) {
      for (int c = rank + csub * nranks; c < BN; c += kProducerWarps * nranks) {
        // the adds stay in rank order, so the sum does not depend on timing
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (PUSH) {
          const int idx = c / nranks;
          float4 part[8];
#pragma unroll
          for (int r = 0; r < 8; ++r)
            part[r] = r < nranks ? *reinterpret_cast<const float4*>(recv + (size_t)(r * cpo + idx) * kBM + r4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            acc.x += part[r].x; acc.y += part[r].y; acc.z += part[r].z; acc.w += part[r].w;
          }
        } else {
          acc = *reinterpret_cast<const float4*>(my_part + c * kBM + r4);
        }
        epi_row(p, rows, blockIdx.x, m0 + c, s_rowf[c], acc, tid & 31);
      }
    }
    // nobody reads or writes a peer's shared memory after the barrier above: a CTA may leave as soon as it is done
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kProducerWarps + 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
}

// ---- activation preparation: optional RMSNorm, split into three bf16 planes ------------------------------------
// Planes hold y = x * norm_weight (or x); the row factor 1/rms (or 1) is written to row_scale for the GEMM epilogue.
__device__ __forceinline__ void store_planes4(unsigned short* base, size_t plane_stride, size_t off, const float* y) {
  unsigned short a[4], b[4], c[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) split3(y[j], a[j], b[j], c[j]);
  *reinterpret_cast<uint2*>(base + off) = make_uint2((uint32_t)a[0] | ((uint32_t)a[1] << 16), (uint32_t)a[2] | ((uint32_t)a[3] << 16));
  *reinterpret_cast<uint2*>(base + plane_stride + off) = make_uint2((uint32_t)b[0] | ((uint32_t)b[1] << 16), (uint32_t)b[2] | ((uint32_t)b[3] << 16));
  *reinterpret_cast<uint2*>(base + 2 * plane_stride + off) = make_uint2((uint32_t)c[0] | ((uint32_t)c[1] << 16), (uint32_t)c[2] | ((uint32_t)c[3] << 16));
}

// Register-resident version: one CTA per activation row, the row is read from global memory exactly once
// (VPT float4 per thread), one block reduction for the sum of squares, one vectorised write per plane.
template <int VPT>
__global__ void __launch_bounds__(256) act_split_reg_kernel(const float* __restrict__ x, size_t x_stride,
                                                            const float* __restrict__ norm_weight, float eps, int K,
                                                            __nv_bfloat16* __restrict__ planes, size_t plane_stride,
                                                            float* __restrict__ row_scale) {
  __shared__ float red[8];
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
      row_scale[m] = 1.0f / sqrtf(t / (float)K + eps);
    }
  } else if (tid == 0) {
    row_scale[m] = 1.0f;
  }
  unsigned short* base = reinterpret_cast<unsigned short*>(planes);
  const float4* nw = reinterpret_cast<const float4*>(norm_weight);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = tid + i * 256;
    if (idx < n4) {
      float y[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      if (norm_weight) {
        const float4 w = __ldg(nw + idx);
        y[0] *= w.x; y[1] *= w.y; y[2] *= w.z; y[3] *= w.w;
      }
      store_planes4(base, plane_stride, (size_t)m * K + (size_t)idx * 4, y);
    }
  }
}

// General version (any K, any alignment of x).
__global__ void __launch_bounds__(256) act_split_kernel(const float* __restrict__ x, size_t x_stride,
                                                        const float* __restrict__ norm_weight, float eps, int K,
                                                        __nv_bfloat16* __restrict__ planes, size_t plane_stride,
                                                        float* __restrict__ row_scale) {
  __shared__ float red[8];
  pi_grid_dependency_wait();
  const int m = blockIdx.x, tid = threadIdx.x;
  const float* row = x + (size_t)m * x_stride;
  if (norm_weight) {
    float ss = 0.f;
    for (int k = tid; k < K; k += blockDim.x) ss = fmaf(row[k], row[k], ss);
    ss = pi_warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
      row_scale[m] = 1.0f / sqrtf(t / (float)K + eps);
    }
  } else if (tid == 0) {
    row_scale[m] = 1.0f;
  }
  unsigned short* base = reinterpret_cast<unsigned short*>(planes);
  for (int k = tid; k < K; k += blockDim.x) {
    const float y = norm_weight ? row[k] * norm_weight[k] : row[k];
    unsigned short a, b, c;
    split3(y, a, b, c);
    const size_t off = (size_t)m * K + k;
    base[off] = a;
    base[plane_stride + off] = b;
    base[2 * plane_stride + off] = c;
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


// Dynamic shared memory of an instantiation: the pipeline stages, the receive area of the cluster reduction (PUSH: up
// to BN + 7 columns of 128 rows, rounded up), alignment slack; never less than what keeps two CTAs off one SM.
template <int BN, int STAGES, bool PUSH>
constexpr size_t ta_smem_bytes() {
  return std::max((size_t)STAGES * (2 * kPlanes * BN * 128) + (PUSH ? (size_t)(BN + 8) * kBM * sizeof(float) : 0) + 1024, kMinSmem);
}

template <int BN, int STAGES, bool PUSH>
cudaError_t launch_ta(pi_ctx* ctx, const GemmParams& p, const CUtensorMap& act, dim3 grid) {
  constexpr size_t smem = ta_smem_bytes<BN, STAGES, PUSH>();
  auto k = gemm_ta_kernel<BN, STAGES, PUSH>;
  static pi_smem_grant granted;  // per instantiation
  if (smem > granted.of(ctx)) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    granted.of(ctx) = smem;
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

// How many clusters of `ksplit` CTAs of this kernel the device can hold at once (clusters are placed inside one GPC,
// so this is less than SMs / ksplit); asked once per cluster size.
template <int BN, int STAGES, bool PUSH>
int max_clusters(pi_ctx* ctx, int ksplit) {
  static int cached[9] = {};
  if (ksplit < 2 || ksplit > 8) return ctx->sm_count;
  if (!cached[ksplit]) {
    constexpr size_t smem = ta_smem_bytes<BN, STAGES, PUSH>();
    auto k = gemm_ta_kernel<BN, STAGES, PUSH>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, ksplit, 1);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ksplit;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, k, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = std::max(1, ctx->sm_count / ksplit / 2);   // conservative
    }
    cached[ksplit] = n;
  }
  return cached[ksplit];
}

int max_clusters_bn(pi_ctx* ctx, int BN, int ksplit) {
  switch (BN) {
    case 16: return max_clusters<16, 6, true>(ctx, ksplit);
    case 32: return max_clusters<32, 6, true>(ctx, ksplit);
    default: return max_clusters<64, 3, true>(ctx, ksplit);
  }
}

// K splits: as many as still run as ONE wave (a CTA owns its SM, so a second, partly filled wave would cost a
// whole extra prologue + epilogue): the tiles' clusters must all be resident at once.  At least two K blocks each.
int pick_ksplit(pi_ctx* ctx, int BN, int tiles, int nkb) {
  for (int ksplit = 8; ksplit >= 2; --ksplit)   // a portable cluster holds up to 8 CTAs; any size below works
    if (nkb / ksplit >= 2 && tiles * ksplit <= ctx->sm_count && tiles <= max_clusters_bn(ctx, BN, ksplit)) return ksplit;
  return 1;
}

}  // namespace

namespace pi_tc {

int pick_bn(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }

pi_status build_gemm_params(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, const pi_act_planes& in, int BN,
                            GemmParams* out, CUtensorMap* map) {
  const int M = a.M, K = (int)lin->cols, N = (int)lin->rows;
  const int rtiles = (N + kBM - 1) / kBM;
  const int nkb = K / kBK;
  PI_REQUIRE(ctx, in.K == K && in.base, "activation planes do not match the projection (%d columns, planes of %d)", K, in.K);

  // one map over the three planes: {K, M rows (rows past M read as zero), 3 planes plane_stride apart}
  {
    const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, (cuuint64_t)kPlanes};
    const cuuint64_t strides[2] = {(cuuint64_t)K * sizeof(__nv_bfloat16), (cuuint64_t)in.plane_stride * sizeof(__nv_bfloat16)};
    const cuuint32_t box[3] = {64, (cuuint32_t)BN, (cuuint32_t)kPlanes};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_tiled()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)in.base, dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return pi_fail(ctx, PI_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  }

  GemmParams pp = {};
  GemmParams& p = pp;
  p.W = static_cast<const int8_t*>(lin->w);
  p.scales = lin->scales;
  p.out = a.out;
  p.ld = lin->ld;
  p.out_stride = a.out_stride;
  p.N = N;
  p.K = K;
  p.M = M;
  p.ksplit = 1;
  p.nkb = nkb;
  p.epi = a.epi;
  if (a.n_out_also > 0) {
    PI_REQUIRE(ctx, a.epi == PI_EPI_STORE && !a.emit && !a.rope && N % 4 == 0 && a.out_stride % 4 == 0 && (uintptr_t)a.out % 16 == 0 &&
                        a.n_out_also <= 8,
               "extra store targets need a plain store epilogue over whole 16-byte groups");
    p.n_out_also = a.n_out_also;
    for (int i = 0; i < a.n_out_also; ++i) {
      PI_REQUIRE(ctx, a.out_also[i] && (uintptr_t)a.out_also[i] % 16 == 0, "extra store target %d is null or misaligned", i);
      p.out_also[i] = a.out_also[i];
    }
  }
  p.err_flag = ctx->dev_err;
  p.act_scale = in.row_scale;
  p.sumsq_in = in.row_scale ? nullptr : (in.sumsq_tiles > 0 ? in.sumsq : nullptr);
  p.sumsq_tiles = in.sumsq_tiles;
  p.sumsq_stride = in.sumsq_stride;
  p.eps = in.eps;
  if (a.emit) {
    pi_act_planes* e = a.emit;
    const int cols_out = a.epi == PI_EPI_SWIGLU ? N / 2 : N;
    PI_REQUIRE(ctx, pi_gemm_tc_can_emit(ctx, lin, a, a.emit_norm_weight != nullptr) && e->base && e->K == cols_out &&
                        e->plane_stride % 4 == 0 && (uintptr_t)e->base % 8 == 0,
               "this launch cannot emit activation planes");
    p.emit_base = e->base;
    p.emit_plane_stride = e->plane_stride;
    p.emit_k = e->K;
    p.emit_norm = a.emit_norm_weight;
    e->row_scale = nullptr;
    if (a.emit_norm_weight) {
      PI_REQUIRE(ctx, e->sumsq && e->sumsq_stride >= (size_t)M, "emit with a norm weight needs a sums-of-squares buffer");
      p.emit_sumsq = e->sumsq;
      p.emit_sumsq_stride = e->sumsq_stride;
      e->sumsq_tiles = rtiles;
      e->eps = a.emit_norm_eps;
    } else {
      e->sumsq_tiles = 0;
    }
  }
  if (a.rope) {
    const pi_rope_kv& r = *a.rope;
    PI_REQUIRE(ctx, pi_gemm_tc_can_rope(ctx, lin, a, r), "this launch cannot fold the rotary embedding and the KV write in");
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
  *out = p;
  return PI_OK;
}

}  // namespace pi_tc

namespace {

// The GEMM proper over activations that already are planes.
pi_status run_gemm(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, const pi_act_planes& in) {
  const int M = a.M, K = (int)lin->cols, N = (int)lin->rows;
  const int BN = pick_bn(M);
  const int mtiles = (M + BN - 1) / BN;
  const int rtiles = (N + kBM - 1) / kBM;
  GemmParams p;
  CUtensorMap map;
  PI_TRY(build_gemm_params(ctx, lin, a, in, BN, &p, &map));
  const int ksplit = pick_ksplit(ctx, BN, rtiles * mtiles, K / kBK);
  p.ksplit = ksplit;
  const dim3 grid(rtiles, ksplit, mtiles);
  cudaError_t err;
  // K split over a cluster: the instantiation with the receive area of the reduction (at 64 activation rows one stage
  // less, a CTA of such a launch has few K blocks anyway)
  if (ksplit > 1) {
    switch (BN) {
      case 16: err = launch_ta<16, 6, true>(ctx, p, map, grid); break;
      case 32: err = launch_ta<32, 6, true>(ctx, p, map, grid); break;
      default: err = launch_ta<64, 3, true>(ctx, p, map, grid); break;
    }
  } else {
    switch (BN) {
      case 16: err = launch_ta<16, 6, false>(ctx, p, map, grid); break;
      case 32: err = launch_ta<32, 6, false>(ctx, p, map, grid); break;
      default: err = launch_ta<64, 4, false>(ctx, p, map, grid); break;
    }
  }
  if (err != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "tensor-core GEMM launch failed: %s", cudaGetErrorString(err));
  ctx->launches++;
  return PI_OK;
}

// Scratch layout shared by pi_launch_gemm_tc and pi_linear_apply_noalloc: [3 planes of rows x K bf16 | rows factors].
pi_act_planes planes_in_scratch(void* scratch, int rows, int K) {
  pi_act_planes pl;
  pl.base = static_cast<__nv_bfloat16*>(scratch);
  pl.plane_stride = (size_t)rows * K;
  pl.K = K;
  pl.row_scale = reinterpret_cast<float*>(pl.base + (size_t)kPlanes * rows * K);
  return pl;
}

}  // namespace

bool pi_gemm_tc_supported(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a) {
  (void)ctx;
  if (lin->kind != PI_INT8) return false;
  if (lin->cols % kBK != 0 || lin->ld != lin->cols) return false;   // whole K blocks, 32-byte aligned rows
  if ((uintptr_t)lin->w % 32 != 0) return false;
  if (lin->rows < 32) return false;
  if (a.epi == PI_EPI_SWIGLU && (lin->rows % 2) != 0) return false;
  if (lin->cols > 65536 * 2) return false;
  return encode_tiled() != nullptr;
}

bool pi_gemm_tc_will_run(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a) {
  return ctx->opt_tensor_gemm && a.M > ctx->opt_gemv_max_m && pi_gemm_tc_supported(ctx, lin, a);
}

bool pi_gemm_tc_can_emit(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, bool with_norm) {
  if (!pi_gemm_tc_will_run(ctx, lin, a)) return false;
  const int N = (int)lin->rows;
  if (N % 4 != 0) return false;                           // planes are written four (two) columns at a time
  if (with_norm && a.epi == PI_EPI_SWIGLU) return false;  // sums of squares of a SwiGLU output are not produced
  return true;
}

bool pi_gemm_tc_can_rope(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, const pi_rope_kv& r) {
  if (!pi_gemm_tc_will_run(ctx, lin, a) || a.epi != PI_EPI_STORE || a.emit) return false;
  if (!r.pool || !r.batch || !r.rope_cos || !r.rope_sin) return false;
  if (r.head_dim != 64 && r.head_dim != 128) return false;            // a 128-row tile is whole heads
  if (r.pool->L.head_dim != r.head_dim || r.pool->L.num_kv_heads != r.num_kv_heads) return false;
  const size_t q_rows = (size_t)r.num_heads * r.head_dim, kv_rows = (size_t)r.num_kv_heads * r.head_dim;
  if (q_rows % kBM != 0 || kv_rows % kBM != 0) return false;          // a tile is all q, all k or all v
  if (lin->rows != q_rows + 2 * kv_rows) return false;
  if ((uintptr_t)a.out % 16 != 0 || a.out_stride % 4 != 0) return false;
  return r.style == 0 || r.style == 1;
}

pi_status pi_launch_act_split(pi_ctx* ctx, const float* x, size_t x_stride, const float* norm_weight, float eps, int M, int K,
                              pi_act_planes* dst) {
  PI_REQUIRE(ctx, dst && dst->base && dst->row_scale && dst->K == K, "activation split needs planes of %d columns and a row-factor array", K);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(M);
  cfg.blockDim = dim3(256);
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  cudaError_t e;
  const int n4 = K / 4;
  const bool vec_ok = ((uintptr_t)x % 16 == 0) && (x_stride % 4 == 0) && (K % 4 == 0) && (dst->plane_stride % 4 == 0) &&
                      ((uintptr_t)dst->base % 8 == 0) && (!norm_weight || (uintptr_t)norm_weight % 16 == 0) && n4 <= 256 * 16;
  if (vec_ok) {  // the row fits the registers of one CTA: single pass
    if (n4 <= 256 * 2) e = cudaLaunchKernelEx(&cfg, act_split_reg_kernel<2>, x, x_stride, norm_weight, eps, K, dst->base, dst->plane_stride, dst->row_scale);
    else if (n4 <= 256 * 4) e = cudaLaunchKernelEx(&cfg, act_split_reg_kernel<4>, x, x_stride, norm_weight, eps, K, dst->base, dst->plane_stride, dst->row_scale);
    else if (n4 <= 256 * 8) e = cudaLaunchKernelEx(&cfg, act_split_reg_kernel<8>, x, x_stride, norm_weight, eps, K, dst->base, dst->plane_stride, dst->row_scale);
    else e = cudaLaunchKernelEx(&cfg, act_split_reg_kernel<16>, x, x_stride, norm_weight, eps, K, dst->base, dst->plane_stride, dst->row_scale);
  } else {
    e = cudaLaunchKernelEx(&cfg, act_split_kernel, x, x_stride, norm_weight, eps, K, dst->base, dst->plane_stride, dst->row_scale);
  }
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "activation split launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  dst->sumsq_tiles = 0;
  return PI_OK;
}

pi_status pi_launch_gemm_tc(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a) {
  PI_REQUIRE(ctx, pi_gemm_tc_supported(ctx, lin, a), "tensor-core GEMM does not support this projection");
  if (a.in_planes) {
    pi_prof_scope prof(ctx, PI_PROF_GEMM_TC);
    return run_gemm(ctx, lin, a, *a.in_planes);
  }
  const int M = a.M, K = (int)lin->cols;
  // scratch (global memory beyond the inputs and outputs): the planes and the row factors
  PI_TRY(pi_reserve(ctx, &ctx->gemm_act, (size_t)kPlanes * M * K * sizeof(__nv_bfloat16) + (size_t)M * sizeof(float) + 256));
  pi_act_planes pl = planes_in_scratch(ctx->gemm_act.ptr, M, K);
  {
    pi_prof_scope prof(ctx, PI_PROF_OTHER);
    PI_TRY(pi_launch_act_split(ctx, a.x, a.x_stride, a.norm_weight, a.norm_eps, M, K, &pl));
  }
  pi_prof_scope prof(ctx, PI_PROF_GEMM_TC);
  return run_gemm(ctx, lin, a, pl);
}

// ---- pi_linear_apply_noalloc -----------------------------------------------------------------------------------
//
// The tensor-core projection needs scratch in global memory: the three bf16 planes the f32 activations are split
// into, plus one factor per activation row.  pi_linear_apply takes that scratch from a buffer the context grows
// with cudaMalloc on demand.  Some callers must not allocate at the moment they run a projection: a serving loop
// that is inside a CUDA stream capture (cudaMalloc is not a capturable operation and invalidates the capture), a
// host thread with a latency budget that a driver allocation (which can take the device-wide allocation lock and
// synchronise) would break, or an embedder that has handed all device memory to its own pool.  For them the same
// kernels run here against a fixed scratch area that is part of the library image: every GPU that loads the
// library carries kNoAllocScratchBytes (about 3 MiB) of it until the process exits.
//
// Limits: int8 projections the tensor path supports (columns a multiple of 128), 1 <= M <= 64 activation rows,
// columns <= 8192.  Larger shapes are refused with PI_ERR_INVALID_ARG; they are never silently routed elsewhere.
//
// The area is shared by every call on the device and keeps whatever the previous call left in it.  Nothing in it
// has to start at zero: rows [0, M) of the planes and the M factors are rewritten by every call before they are
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
    (size_t)kPlanes * kNoAllocMaxM * kNoAllocMaxK * sizeof(__nv_bfloat16) + (size_t)kNoAllocMaxM * sizeof(float) + 256;
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
  PI_ENTER(ctx);
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
  pi_act_planes pl = planes_in_scratch(scratch, M, (int)lin->cols);
  PI_TRY(pi_launch_act_split(ctx, x_dev, lin->cols, nullptr, 0.f, M, (int)lin->cols, &pl));
  return run_gemm(ctx, lin, a, pl);
}
