// A chain of dequant projections in ONE persistent launch (batches of up to 64 activation rows).
//
// A decode step is a chain of dependent projections with nothing between them but their own epilogues:
// o -> [gate;up] -> down -> next layer's [q;k;v] (-> LM head after the last layer).  Launched one by one, each pays a
// launch hop, a prologue (TMEM allocation, barriers, first weight loads), idle SMs when its row tiles do not fill
// the machine, and a tear-down.  Here up to four consecutive projections ("phases") run in one grid of one CTA per
// SM that stays resident for all of them:
//
//   * every phase's work is its (row tile, K block) units in row-tile-major order, cut into equal contiguous shares,
//     one per CTA - a wide matrix ([gate;up]: 88 row tiles) and a narrow one (o, down: 16) both keep all SMs busy;
//   * a CTA's share is a few "segments" (a K range of one row tile).  Tensor memory holds the accumulators of two
//     segments, so the tensor pipe runs through a share that crosses a tile boundary without waiting for an
//     epilogue; the accumulators are taken out when the share ends (or after two segments);
//   * a segment that covers a tile's whole K range goes through shared memory straight to the epilogue.  Otherwise
//     the raw partial tile goes to a scratch slot in global memory, and once every CTA that holds a part of the tile
//     has handed its part in, each of them adds up - IN SLOT (= K) ORDER, whoever does it - and finishes its own
//     slice of the tile's activation rows: one round trip of loads per CTA, results that do not depend on timing;
//   * between phases a grid-wide barrier (a counter in global memory that only grows: arriving is one fire-and-forget
//     reduction, waiting is polling for this launch's target); a CTA's weight producers do not wait
//     for it - the next phase's weights are already on their way into registers and tensor memory while the barrier
//     is pending; only the activation loads (TMA) of the next phase do;
//   * TMEM, the mbarriers and the pipeline state are set up once.
//
// The inner machinery is that of the single-projection kernel (pi_gemm_tc.cu): swap-AB tcgen05.mma kind::f16 with
// the widened int8 weights as the A operand in tensor memory, the activations as three exact bf16 planes fetched by
// one 3-D TMA box per K atom, f32 accumulation in tensor memory, and the same epilogues (pi_gemm_tc.cuh).  Every
// wait is bounded; a wait that runs out raises the context's error word and the kernel winds down.
//
// Replaces math::matmat_i8_weight_parallel + transpose_rb_to_br (reference src/math.rs:223-290) for the batched
// decode step, with math::rms_norm (src/math.rs:4-22), the rotary embedding and KV write (src/model.rs:1065-1107),
// SwiGLU and the residual adds (src/model.rs:1127-1167) folded into the epilogues.
#include <stdlib.h>

#include <algorithm>
#include <new>

#include "pi_gemm_tc.cuh"

namespace {
using namespace pi_tc;

constexpr int kMaxPhases = 4;
constexpr uint32_t kGridSpinLimit = 1u << 22;   // polls, 32 ns apart

// Optional per-CTA timeline (compile with -DPI_CHAIN_TRACE): %globaltimer stamps of the steps of every phase, written
// to a buffer that the launcher dumps to the file named by the environment variable PI_CHAIN_TRACE_FILE.
#ifdef PI_CHAIN_TRACE
#define PI_TRACE(cp, cta, slot)                                                             \
  do {                                                                                      \
    unsigned long long _t;                                                                  \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t));                                  \
    (cp).trace[(size_t)(cta) * 64 + (slot)] = _t;                                           \
  } while (0)
#define PI_TRACE_FIRST(cp, cta, slot)     /* once per phase: `trace_seen` is a local bit mask of phases */ \
  do {                                                                                      \
    const int _ph = ((slot) - 8) / 12;                                                      \
    if (!(trace_seen & (1u << _ph))) {                                                      \
      trace_seen |= 1u << _ph;                                                              \
      PI_TRACE(cp, cta, slot);                                                              \
    }                                                                                       \
  } while (0)
#else
#define PI_TRACE(cp, cta, slot) do { } while (0)
#define PI_TRACE_FIRST(cp, cta, slot) do { } while (0)
#endif

struct ChainParams {
#ifdef PI_CHAIN_TRACE
  unsigned long long* trace;  // [grid][64]
#endif
  GemmParams ph[kMaxPhases];
  int rtiles[kMaxPhases];
  int active[kMaxPhases];     // CTAs that own units of the phase: min(grid, units)
  int nphases;
  float* partials;            // [slots][BN][128] raw partial tiles
  unsigned int* tickets;      // [2][max_tiles] parts handed in per row tile; zero between uses; phase ph uses half ph & 1
  unsigned int* done;         // [2][max_tiles] holders of a part that have finished their slice; zero between uses
  int max_tiles;
  unsigned int* bar_count;    // [phases] x 32 words: arrivals at the barrier after each phase since the buffer was cleared
  int* err_flag;
};
struct ChainMaps {
  CUtensorMap m[kMaxPhases];
};

// This CTA's units, phase after phase.
struct UnitIter {
  int ph;      // phase of the current unit; nphases at the end
  int tile, kb;
  int left;    // units left in this CTA's share of the phase, the current one included
  int nkb;
  bool first;  // the current unit opens a segment
};

__device__ __forceinline__ void iter_enter(UnitIter& it, const ChainParams& cp, int cta) {
  while (it.ph < cp.nphases) {
    const int nkb = cp.ph[it.ph].nkb, act = cp.active[it.ph];
    if (cta < act) {
      const long U = (long)cp.rtiles[it.ph] * nkb;
      const long u0 = U * cta / act, u1 = U * (cta + 1) / act;
      it.nkb = nkb;
      it.tile = (int)(u0 / nkb);
      it.kb = (int)(u0 - (long)it.tile * nkb);
      it.left = (int)(u1 - u0);
      it.first = true;
      return;
    }
    ++it.ph;
  }
}
__device__ __forceinline__ bool iter_seg_last(const UnitIter& it) { return it.left == 1 || it.kb == it.nkb - 1; }
__device__ __forceinline__ void iter_next(UnitIter& it, const ChainParams& cp, int cta) {
  it.first = iter_seg_last(it);
  --it.left;
  ++it.kb;
  if (it.left == 0) {
    ++it.ph;
    iter_enter(it, cp, cta);
    return;
  }
  if (it.kb == it.nkb) {
    it.kb = 0;
    ++it.tile;
  }
}
// The CTA whose share holds unit x of a phase with U units cut into `act` shares (share c = [U*c/act, U*(c+1)/act)).
__device__ __forceinline__ int owner_of(long x, long U, int act) { return (int)(((x + 1) * act - 1) / U); }

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Fire-and-forget arrival: orders this thread's earlier writes (and, after a CTA barrier and a fence, its CTA's) before
// the increment becomes visible; nothing comes back, so the thread does not wait for the round trip.
__device__ __forceinline__ void red_add_release(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait on an mbarrier; polls are only counted once the grid dependency of this launch is resolved (until
// then nothing can make progress and the wait is the preceding kernel's, however long that runs).
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

// What the epilogues need from their CTA.
struct EpiCtx {
  float* my_part;            // [BN][128] shared
  float* s_rowf;             // [BN] shared
  volatile int* s_abort;
  volatile int* s_dep_ok;
  uint32_t accum_full, accum_empty;   // mbarriers
  uint32_t tmem_d;           // accumulator base (lane 0, column 0)
  int cta;
};

constexpr int kMaxSegs = 2;   // segment accumulators (three column groups each) that tensor memory holds

// A run of segments whose accumulators are waiting in tensor memory: consecutive row tiles t0 .. t0 + nseg - 1 of one
// phase; the first starts at K block kb0, the last ends with K block kb_last, the ones between cover all of K.
struct SegBatch {
  int ph, t0, nseg, kb0, kb_last;
};

__device__ __forceinline__ bool seg_whole(const SegBatch& b, int j, int nkb) {
  return (j > 0 || b.kb0 == 0) && (j < b.nseg - 1 || b.kb_last == nkb - 1);
}

// Which CTAs hold a part of row tile `tile`: [first, first + n).
__device__ __forceinline__ void tile_holders(const ChainParams& cp, int ph, int tile, int* first, int* n) {
  const int nkb = cp.ph[ph].nkb;
  const long U = (long)cp.rtiles[ph] * nkb;
  const int act = cp.active[ph];
  const int c0 = owner_of((long)tile * nkb, U, act), c1 = owner_of((long)(tile + 1) * nkb - 1, U, act);
  *first = c0;
  *n = c1 - c0 + 1;
}

// Take the accumulators of a batch of segments out of tensor memory.  All 16 producer warps call this in lock step
// (named barrier 1).  Partial tiles go to their scratch slots first and are handed in at once (a ticket per tile,
// fire and forget), so that the other holders of those tiles are not kept waiting; whole tiles then go through shared
// memory, one after the other, to their epilogue.  Out of line on purpose: it would otherwise be cloned into every
// slot of the unrolled producer loop.
template <int BN>
__device__ __noinline__ void batch_drain(const ChainParams& cp, const EpiCtx& e, SegBatch b, int batch_no) {
  constexpr int kTileFloats = BN * kBM;
  constexpr int kColsPerHalf = BN / 2 >= 16 ? BN / 2 : 16;  // BN 16: only the first half works
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = warp & 3, half = (warp >> 2) & 1;
  const GemmParams& p = cp.ph[b.ph];
  const bool drainer = warp < kParkWarps && (BN >= 32 || half == 0);
  int got = 0;
  if (warp < kParkWarps) {
    if (lane == 0) {
      got = (!*e.s_abort && mbar_wait_dep(e.accum_full, (uint32_t)(batch_no & 1), e.s_dep_ok)) ? 1 : 0;
      if (!got && !*e.s_abort) {
        *e.s_abort = 1;
        if (cp.err_flag) atomicExch(cp.err_flag, 5);
      }
    }
    got = __shfl_sync(0xffffffffu, got, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // The accumulate is over, so the phase before this one is complete: the row factors (1/rms from the sums of
    // squares that phase emitted) can be read now.  Their readers come after the next named barrier.
    if (tid < BN) e.s_rowf[tid] = act_row_factor(p, tid);
  }
  // accumulator of segment j (three groups of BN columns from column j * 3 * BN, added) -> dst[c][128 rows]
  auto drain = [&](int j, float* dst) {
    const uint32_t my_d = e.tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)(j * kPlanes * BN);
#pragma unroll 1
    for (int c0 = half * kColsPerHalf; c0 < (half + 1) * kColsPerHalf && c0 < BN; c0 += 16) {
      float v[16];
      if (got) {
        tmem_ld_sum16<BN>(my_d, c0, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) dst[(c0 + i) * kBM + quad * 32 + lane] = v[i];
    }
  };
  // 1. partial tiles: scratch slot (cta + tile), then one ticket per tile
  bool any_partial = false;
  for (int j = 0; j < b.nseg; ++j) {
    if (seg_whole(b, j, p.nkb)) continue;
    any_partial = true;
    if (drainer) drain(j, cp.partials + (size_t)(e.cta + b.t0 + j) * kTileFloats);
  }
  if (any_partial && drainer) __threadfence();
  asm volatile("bar.sync 1, %0;" ::"n"(kProducerWarps * 32) : "memory");   // parts are out, s_rowf is written
  if (any_partial && tid == 0) {
    unsigned int* tk = cp.tickets + (size_t)(b.ph & 1) * cp.max_tiles;
    for (int j = 0; j < b.nseg; ++j)
      if (!seg_whole(b, j, p.nkb)) red_add_release(tk + b.t0 + j, 1u);
    PI_TRACE(cp, e.cta, 8 + b.ph * 12 + 6);
  }
  // 2. whole tiles: through shared memory to the epilogue
  for (int j = 0; j < b.nseg; ++j) {
    if (!seg_whole(b, j, p.nkb)) continue;
    const int tile = b.t0 + j;
    if (drainer) drain(j, e.my_part);
    EpiRows rows;
    epi_rows_load(p, tile * kBM, tid, rows);
    asm volatile("bar.sync 1, %0;" ::"n"(kProducerWarps * 32) : "memory");
    for (int c = warp; c < BN; c += kProducerWarps)
      epi_row(p, rows, tile, c, e.s_rowf[c], *reinterpret_cast<const float4*>(e.my_part + c * kBM + lane * 4), lane);
    asm volatile("bar.sync 1, %0;" ::"n"(kProducerWarps * 32) : "memory");   // my_part is free again
  }
  // 3. every accumulator of the batch has been read: the tensor pipe may overwrite them
  if (drainer) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(e.accum_empty);
  }
}

// The end of this CTA's share of a phase: the row tiles it holds only a part of (its first and/or its last) are finished
// together with the other holders.  Each holder waits until all parts of the tile are handed in (bounded), then adds
// up and finishes the activation rows c = its index among the holders, + their number, ...; the sum runs over the
// slots in K order, so it is the same whoever computes it.  The last holder to finish clears the tile's counters
// (their half of the counter arrays is not used again before the phase after the next).
template <int BN>
__device__ __noinline__ void share_finish(const ChainParams& cp, const EpiCtx& e, int ph, int tile_a, int tile_b) {
  constexpr int kTileFloats = BN * kBM;
  __shared__ int s_ok;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const GemmParams& p = cp.ph[ph];
  unsigned int* tk = cp.tickets + (size_t)(ph & 1) * cp.max_tiles;
  unsigned int* dn = cp.done + (size_t)(ph & 1) * cp.max_tiles;
  int first[2] = {0, 0}, n[2] = {0, 0};
  const int tiles[2] = {tile_a, tile_b};
  for (int k = 0; k < 2; ++k)
    if (tiles[k] >= 0) tile_holders(cp, ph, tiles[k], &first[k], &n[k]);
  if (tid == 0) {   // both tiles' parts are waited for together
    int ok = 0;
    for (uint32_t spin = 0; spin < kGridSpinLimit; ++spin) {
      const bool a = tiles[0] < 0 || ld_acquire_u32(tk + tiles[0]) >= (unsigned int)n[0];
      const bool b = tiles[1] < 0 || ld_acquire_u32(tk + tiles[1]) >= (unsigned int)n[1];
      if (a && b) {
        ok = 1;
        break;
      }
      if (*e.s_abort) break;
      __nanosleep(20);
    }
    if (!ok && !*e.s_abort) {
      *e.s_abort = 1;
      if (cp.err_flag) atomicExch(cp.err_flag, 8);
    }
    s_ok = ok;
    PI_TRACE(cp, e.cta, 8 + ph * 12 + 7);
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kProducerWarps * 32) : "memory");
  if (s_ok) {
    __threadfence();
    for (int k = 0; k < 2; ++k) {
      const int tile = tiles[k];
      if (tile < 0) continue;
      EpiRows rows;
      epi_rows_load(p, tile * kBM, tid, rows);
      const int mine = e.cta - first[k], nn = n[k];
      const float* slot0 = cp.partials + (size_t)(first[k] + tile) * kTileFloats + lane * 4;
      for (int c = mine + warp * nn; c < BN; c += kProducerWarps * nn) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int j = 0; j < nn; ++j) {   // slot order = K order
          const float4 v = __ldcg(reinterpret_cast<const float4*>(slot0 + (size_t)j * kTileFloats + c * kBM));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        epi_row(p, rows, tile, c, e.s_rowf[c], acc, lane);
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kProducerWarps * 32) : "memory");
  // Every thread of this CTA has read all parts.  A side thread counts the holders that are through and the last one
  // clears the counters; nobody waits for that round trip (warp 1 meets it at its next use of the value only).
  if (tid == 32)
    for (int k = 0; k < 2; ++k) {
      if (tiles[k] < 0) continue;
      unsigned int d;
      asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(d) : "l"(dn + tiles[k]), "r"(1u) : "memory");
      if (d == (unsigned int)n[k] - 1u) {
        tk[tiles[k]] = 0u;
        dn[tiles[k]] = 0u;
      }
    }
}

template <int BN, int SA, int SB>
__global__ void __launch_bounds__(kThreads, 1)
gemm_chain_kernel(const __grid_constant__ ChainParams cp, const __grid_constant__ ChainMaps maps) {
  constexpr int kBAtomBytes = kPlanes * BN * 128;           // one 64-element K atom: BN rows of plane 0, 1, 2
  constexpr int kBStageBytes = 2 * kBAtomBytes;
  constexpr int kSegCols = kPlanes * BN;                     // one segment's accumulator: W*p0 | W*p1 | W*p2
  constexpr int kDCols = kMaxSegs * kSegCols;
  constexpr int kAStart = (kDCols + 63) / 64 * 64;          // weight stages start on a 64-column boundary
  static_assert(kSegCols <= 256, "one MMA covers at most 256 accumulator columns");
  static_assert(kAStart + SA * kACols <= 512, "TMEM holds 512 columns");
  constexpr int kTmemCols = 512;
  constexpr int kEpiWarps = BN >= 32 ? kParkWarps : 4;      // warps that move the accumulators out of TMEM
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // mbarriers: weights in tensor memory (full / empty per A stage), activations in shared memory (per B stage), accumulators
  __shared__ __align__(8) unsigned long long bars[2 * SA + 2 * SB + 2];
  __shared__ uint32_t s_tmem;
  __shared__ volatile unsigned int s_base[kMaxPhases];   // barrier counters before this launch began
  __shared__ volatile int s_abort;
  __shared__ volatile int s_dep_ok;   // the preceding kernel has completed and s_base is recorded
  __shared__ float s_rowf[BN];        // row factor of the activation rows

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = warp & 3, kq = (warp >> 2) & 3;
  const int cta = blockIdx.x, G = gridDim.x;
#ifdef PI_CHAIN_TRACE
  unsigned int trace_seen = 0;
#endif
  const uint32_t a_full0 = smem_u32(&bars[0]), a_empty0 = smem_u32(&bars[SA]);
  const uint32_t b_full0 = smem_u32(&bars[2 * SA]), b_empty0 = smem_u32(&bars[2 * SA + SB]);
  const uint32_t accum_full = smem_u32(&bars[2 * SA + 2 * SB]), accum_empty = smem_u32(&bars[2 * SA + 2 * SB + 1]);
  float* my_part = reinterpret_cast<float*>(smem + SB * kBStageBytes);   // [BN][128], apart from the B stages
  pi_grid_launch_dependents();
  if (tid == 0) PI_TRACE(cp, cta, 0);

  // ---- weight producers: the first loads go out before anything else (weights depend on nothing) ----------------
  // Rolling prefetch: the 32 bytes of unit i + 4 are requested into the register slot that unit i has just left.
  constexpr int kGroup = 4;
  uint32_t cur[kGroup][8];
  UnitIter pf;   // prefetch position, four units ahead of the unit being widened
  pf.ph = 0;
  auto unit_ptr = [&](const UnitIter& u) {
    const GemmParams& p = cp.ph[u.ph];
    const int row = min(u.tile * kBM + quad * 32 + lane, p.N - 1);
    return reinterpret_cast<const unsigned char*>(p.W) + (size_t)row * p.ld + (size_t)u.kb * kBK + kq * 32;
  };
  if (warp < kProducerWarps) {
    iter_enter(pf, cp, cta);
#pragma unroll
    for (int d = 0; d < kGroup; ++d)
      if (pf.ph < cp.nphases) {
        ld_stream_32(unit_ptr(pf), &cur[d][0]);
        iter_next(pf, cp, cta);
      }
  }

  if (tid == 0) {
    for (int s = 0; s < SA; ++s) {
      mbar_init(a_full0 + 8 * s, kProducerWarps);          // one arrival per producer warp
      mbar_init(a_empty0 + 8 * s, 1);                      // one tcgen05.commit
    }
    for (int s = 0; s < SB; ++s) {
      mbar_init(b_full0 + 8 * s, 1);                       // the TMA thread's expect_tx
      mbar_init(b_empty0 + 8 * s, 1);                      // one tcgen05.commit
    }
    mbar_init(accum_full, 1);
    mbar_init(accum_empty, kEpiWarps);
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
  const uint32_t tmem = s_tmem;
  const uint32_t tmem_a0 = tmem + (uint32_t)kAStart;
  const uint32_t smem_base = smem_u32(smem);

  // The barrier after phase k is a counter that only grows: every CTA adds one when it is through with the phase, and
  // the barrier is passed once the counter has grown by the size of the grid.  The counters are shared with the
  // preceding launch, which may still be running while this one starts (programmatic dependent launch).  So their
  // values "before this launch" are read only once the preceding kernel has completed (by the TMA lane, which then
  // raises s_dep_ok), and no thread arrives at a barrier before that.
  // Wait until the first `need` barriers of this launch are passed; false when the limit ran out.
  auto grid_wait = [&](int need) {
    if (need <= 0) return true;
    const unsigned int* ctr = cp.bar_count + (size_t)(need - 1) * 32;
    for (uint32_t spin = 0; spin < kGridSpinLimit; ++spin) {
      if (s_dep_ok && (int)(ld_acquire_u32(ctr) - (s_base[need - 1] + (unsigned int)G)) >= 0) return true;
      if (s_abort) return false;
      __nanosleep(32);
    }
    return false;
  };

  if (warp < kProducerWarps) {
    // ================= weight producers + epilogues ================================================================
    UnitIter cu;
    cu.ph = 0;
    iter_enter(cu, cp, cta);
    bool dep_waited = false;
    int it = 0, batch_no = 0;
    int arrived = 0;   // grid barriers this CTA has arrived at (thread 0 only)
    // Arrive at the barriers that end phases [arrived, upto): thread 0, after every thread's stores of the phase (a CTA
    // barrier orders those before this thread's fence).  Each barrier has a counter of its own, so a CTA with nothing
    // to do in a phase need not wait for the barrier before it.
    auto arrive_upto = [&](int upto) {
      upto = min(upto, cp.nphases - 1);   // nothing follows the last phase
      if (arrived >= upto) return;
      for (uint32_t spin = 0; !s_dep_ok && spin < kGridSpinLimit; ++spin) __nanosleep(100);   // the bases are recorded first
      if (!s_dep_ok && !s_abort) {
        s_abort = 1;
        if (cp.err_flag) atomicExch(cp.err_flag, 6);
      }
      asm volatile("fence.proxy.async.global;" ::: "memory");   // the next phase reads these stores through TMA
      __threadfence();
      for (; arrived < upto; ++arrived) red_add_release(cp.bar_count + (size_t)arrived * 32, 1u);
    };
    if (tid == 0) arrive_upto(cu.ph);   // phases in which this CTA has nothing to do

    const uint32_t my_a = tmem_a0 + ((uint32_t)(quad * 32) << 16) + (uint32_t)(kq * 16);
    EpiCtx ec;
    ec.my_part = my_part;
    ec.s_rowf = s_rowf;
    ec.s_abort = &s_abort;
    ec.s_dep_ok = &s_dep_ok;
    ec.accum_full = accum_full;
    ec.accum_empty = accum_empty;
    ec.tmem_d = tmem;
    ec.cta = cta;
    SegBatch batch;     // segments whose accumulators are waiting in tensor memory
    batch.nseg = 0;
    int share_ph = -1, share_t0 = 0, share_kb0 = 0;   // where this CTA's share of the current phase began
    // Once a wait has run out (s_abort) the warps stop waiting and stop feeding the pipeline, but they still walk
    // their units to the end: the named barriers of the epilogues below must be reached by all 16 warps in lock step.
    while (cu.ph < cp.nphases) {
#pragma unroll
      for (int d = 0; d < kGroup; ++d) {
        if (cu.ph >= cp.nphases) break;
        const int s = it % SA;
        if (cu.ph != share_ph) {   // first unit of this CTA's share of a phase
          share_ph = cu.ph;
          share_t0 = cu.tile;
          share_kb0 = cu.kb;
        }
        if (cu.first && batch.nseg == 0) {
          batch.ph = cu.ph;
          batch.t0 = cu.tile;
          batch.kb0 = cu.kb;
        }
        uint32_t h[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) widen4(cur[d][i], h[2 * i], h[2 * i + 1]);
        if (pf.ph < cp.nphases) {
#ifndef PI_CHAIN_DBG_NO_W
          ld_stream_32(unit_ptr(pf), &cur[d][0]);
#endif
          iter_next(pf, cp, cta);
        }
        int ok = 1;
        if (lane == 0) ok = (!s_abort && mbar_wait_dep(a_empty0 + 8 * s, ((it / SA) & 1) ^ 1, &s_dep_ok)) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");   // the MMAs that read this stage are done
          tmem_st16(my_a + (uint32_t)(s * kACols), h);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(a_full0 + 8 * s);
          if (tid == 0) PI_TRACE_FIRST(cp, cta, 8 + cu.ph * 12 + 4);
        } else if (lane == 0 && !s_abort) {
          s_abort = 1;
          if (cp.err_flag) atomicExch(cp.err_flag, 2);
        }
        ++it;

        if (iter_seg_last(cu)) {
          ++batch.nseg;
          batch.kb_last = cu.kb;
          const bool share_end = cu.left == 1;
          if (share_end || batch.nseg == kMaxSegs) {
            // ---- take the pending accumulators out; at the end of the share also finish the split tiles ------------
            if (!dep_waited) {
              asm volatile("griddepcontrol.wait;" ::: "memory");   // the epilogues read what the preceding kernel wrote
              dep_waited = true;
            }
            if (tid == 0) PI_TRACE(cp, cta, 8 + cu.ph * 12 + 5);
            batch_drain<BN>(cp, ec, batch, batch_no);
            ++batch_no;
            batch.nseg = 0;
            if (share_end) {
              const int nkb = cu.nkb;
              const int tile_a = (share_kb0 != 0 || (cu.tile == share_t0 && cu.kb != nkb - 1)) ? share_t0 : -1;
              const int tile_b = (cu.kb != nkb - 1 && cu.tile != share_t0) ? cu.tile : -1;
              if (tile_a >= 0 || tile_b >= 0) share_finish<BN>(cp, ec, cu.ph, tile_a, tile_b);
              asm volatile("fence.proxy.async.global;" ::: "memory");   // the next phase reads these stores through TMA
              asm volatile("bar.sync 1, %0;" ::"n"(kProducerWarps * 32) : "memory");   // every thread's stores are issued
              if (tid == 0) {
                PI_TRACE(cp, cta, 8 + cu.ph * 12 + 8);
                UnitIter nx = cu;
                iter_next(nx, cp, cta);
                arrive_upto(nx.ph);
                PI_TRACE(cp, cta, 8 + cu.ph * 12 + 9);
              }
            }
          }
        }
        iter_next(cu, cp, cta);
      }
    }
    if (tid == 0) arrive_upto(cp.nphases);   // after an abort: keep the barriers consistent for the other CTAs
  } else if (warp == kProducerWarps) {
    // ================= activation loader: one 3-D TMA box {64 K, BN rows, 3 planes} per K atom =====================
    if (lane == 0) {
      UnitIter cu;
      cu.ph = 0;
      iter_enter(cu, cp, cta);
      int it = 0, ready_ph = -1;
      bool issued = false;
      asm volatile("griddepcontrol.wait;" ::: "memory");   // the first phase's planes come from the preceding kernel
      for (int k = 0; k < kMaxPhases; ++k) s_base[k] = ld_acquire_u32(cp.bar_count + (size_t)k * 32);
      __threadfence_block();
      s_dep_ok = 1;
      PI_TRACE(cp, cta, 1);
      while (cu.ph < cp.nphases) {
        if (cu.ph != ready_ph) {
          if (!grid_wait(cu.ph)) {   // every CTA is through with the phases before this one
            if (!s_abort && cp.err_flag) atomicExch(cp.err_flag, 6);
            s_abort = 1;
            break;
          }
          if (cu.ph > 0) asm volatile("fence.proxy.async.global;" ::: "memory");
          ready_ph = cu.ph;
          PI_TRACE(cp, cta, 8 + cu.ph * 12 + 0);
        }
        const int s = it % SB;
        if (s_abort) break;
        if (!mbar_wait_dep(b_empty0 + 8 * s, ((it / SB) & 1) ^ 1, &s_dep_ok)) {
          s_abort = 1;
          if (cp.err_flag) atomicExch(cp.err_flag, 3);
          break;
        }
        const uint32_t bar = b_full0 + 8 * s;
        const uint32_t b_stage = smem_base + s * kBStageBytes;
#ifdef PI_CHAIN_DBG_NO_B
        mbar_arrive(bar);
        if (false)
#else
        mbar_arrive_expect_tx(bar, kBStageBytes);
#endif
#pragma unroll
        for (int atom = 0; atom < 2; ++atom) {
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
                  b_stage + atom * kBAtomBytes),
              "l"(&maps.m[cu.ph]), "r"(bar), "r"(cu.kb * kBK + atom * 64), "r"(0), "r"(0)
              : "memory");
        }
        issued = true;
        PI_TRACE_FIRST(cp, cta, 8 + cu.ph * 12 + 1);
        ++it;
        iter_next(cu, cp, cta);
      }
      if (s_abort && issued)   // copies may still be landing in this CTA's shared memory: give them time before it exits
        for (int i = 0; i < 400; ++i) __nanosleep(100);
    }
  } else {
    // ================= MMA issuer ==================================================================================
    if (lane == 0) {
      // kind::f16, D = f32, A (TMEM) and B (shared, K-major) = bf16, M = 128, N = 3*BN: one MMA per K step leaves
      // W*p0, W*p1, W*p2 in the three column groups of the segment's accumulator
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kSegCols >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      UnitIter cu;
      cu.ph = 0;
      iter_enter(cu, cp, cta);
      int it = 0, nseg = 0, batch_no = 0;
      while (cu.ph < cp.nphases) {
        const int sa = it % SA, sb = it % SB;
        if (cu.first && nseg == 0 && batch_no > 0) {   // the accumulators of the previous batch have been taken out
          if (s_abort || !mbar_wait_dep(accum_empty, (uint32_t)((batch_no - 1) & 1), &s_dep_ok)) {
            if (!s_abort && cp.err_flag) atomicExch(cp.err_flag, 7);
            s_abort = 1;
            break;
          }
        }
        if (s_abort || !mbar_wait_dep(b_full0 + 8 * sb, (it / SB) & 1, &s_dep_ok) ||
            !mbar_wait_dep(a_full0 + 8 * sa, (it / SA) & 1, &s_dep_ok)) {
          if (!s_abort && cp.err_flag) atomicExch(cp.err_flag, 4);
          s_abort = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        PI_TRACE_FIRST(cp, cta, 8 + cu.ph * 12 + 2);
        const uint64_t db0 = smem_desc(smem_base + sb * kBStageBytes);
        const uint32_t a_s = tmem_a0 + (uint32_t)(sa * kACols);
        const uint32_t d_seg = tmem + (uint32_t)(nseg * kSegCols);
#pragma unroll
        for (int atom = 0; atom < 2; ++atom) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {  // 16 K elements: 8 TMEM columns of A, 32 bytes of every B row
            const uint64_t db = db0 + (uint64_t)((atom * kBAtomBytes + ks * 32) >> 4);
            umma_f16_ts(d_seg, a_s + (uint32_t)((atom * 4 + ks) * 8), db, idesc, (!cu.first || atom + ks > 0) ? 1u : 0u);
          }
        }
        umma_commit(a_empty0 + 8 * sa);  // the weight stage (TMEM columns) and the activation stage (shared memory)
        umma_commit(b_empty0 + 8 * sb);  // are free once these MMAs are done
        if (iter_seg_last(cu)) {
          ++nseg;
          if (cu.left == 1 || nseg == kMaxSegs) {
            umma_commit(accum_full);
            PI_TRACE(cp, cta, 8 + cu.ph * 12 + 3);
            nseg = 0;
            ++batch_no;
          }
        }
        ++it;
        iter_next(cu, cp, cta);
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kProducerWarps + 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
}

// ---- host side: the queue of a context ------------------------------------------------------------------------------
struct ChainQueue {
  ChainParams cp = {};
  ChainMaps maps = {};
  int n = 0, BN = 0;
  bool open = false;
  // scratch (global memory beyond the inputs and outputs): partial tiles, tickets, the grid barrier
  void* ws = nullptr;
  size_t ws_slots = 0, ws_tiles = 0;
  int ws_bn = 0;
};

ChainQueue* queue_of(pi_ctx* ctx) {
  if (!ctx->gemm_chain) ctx->gemm_chain = new (std::nothrow) ChainQueue();
  return static_cast<ChainQueue*>(ctx->gemm_chain);
}

template <int BN, int SA, int SB>
cudaError_t launch_chain(pi_ctx* ctx, const ChainQueue& q, int grid) {
  constexpr size_t smem = (size_t)SB * (2 * kPlanes * BN * 128) + (size_t)BN * kBM * sizeof(float) + 1024;
  auto k = gemm_chain_kernel<BN, SA, SB>;
  static pi_smem_grant granted;  // per instantiation
  if (smem > granted.of(ctx)) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    granted.of(ctx) = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, k, q.cp, q.maps);
}

}  // namespace

bool pi_gemm_chain_usable(const pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a) {
  return ctx->opt_gemm_chain && a.M <= 64 && pi_gemm_tc_supported(ctx, lin, a);
}

void pi_gemm_chain_open(pi_ctx* ctx) {
  ChainQueue* q = queue_of(ctx);
  if (q) q->open = true;
}

pi_status pi_gemm_chain_flush(pi_ctx* ctx) {
  ChainQueue* q = static_cast<ChainQueue*>(ctx->gemm_chain);
  if (!q || q->n == 0) return PI_OK;
  pi_prof_scope prof(ctx, PI_PROF_GEMM_TC);
  const int BN = q->BN;
  // one CTA per SM; every phase cuts its units into min(grid, units) shares
  int grid = 1;
  size_t slots = 0, tiles = 0;
  for (int i = 0; i < q->n; ++i) {
    const long U = (long)q->cp.rtiles[i] * q->cp.ph[i].nkb;
    grid = std::max(grid, (int)std::min<long>(U, ctx->sm_count));
  }
  for (int i = 0; i < q->n; ++i) {
    const long U = (long)q->cp.rtiles[i] * q->cp.ph[i].nkb;
    q->cp.active[i] = (int)std::min<long>(U, grid);
    slots = std::max(slots, (size_t)q->cp.active[i] + (size_t)q->cp.rtiles[i]);
    tiles = std::max(tiles, (size_t)q->cp.rtiles[i]);
  }
  q->cp.nphases = q->n;
  q->cp.err_flag = ctx->dev_err;
  const int n = q->n;
  q->n = 0;   // whatever happens below, the queue is empty afterwards
  if (slots > q->ws_slots || tiles > q->ws_tiles || BN > q->ws_bn) {
    // the buffer may still be in use by a queued launch
    PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (q->ws) PI_CUDA(ctx, cudaFree(q->ws));
    q->ws = nullptr;
    q->ws_slots = std::max(slots, q->ws_slots);
    q->ws_tiles = std::max(tiles, q->ws_tiles);
    q->ws_bn = std::max(BN, q->ws_bn);
    const size_t bytes = q->ws_slots * (size_t)q->ws_bn * kBM * sizeof(float) + (4 * q->ws_tiles + 32 * kMaxPhases) * sizeof(unsigned int);
    PI_CUDA(ctx, cudaMalloc(&q->ws, bytes));
    PI_CUDA(ctx, cudaMemsetAsync(q->ws, 0, bytes, ctx->stream));
  }
  q->cp.partials = static_cast<float*>(q->ws);
  unsigned int* words = reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(q->ws) + q->ws_slots * (size_t)q->ws_bn * kBM * sizeof(float));
  q->cp.bar_count = words;          // one 128-byte line per barrier
  q->cp.tickets = words + 32 * kMaxPhases;
  q->cp.done = q->cp.tickets + 2 * q->ws_tiles;
  q->cp.max_tiles = (int)q->ws_tiles;
#ifdef PI_CHAIN_TRACE
  static unsigned long long* trace_dev = nullptr;
  const size_t trace_bytes = (size_t)256 * 64 * sizeof(unsigned long long);
  if (!trace_dev) cudaMalloc(&trace_dev, trace_bytes);
  cudaMemsetAsync(trace_dev, 0, trace_bytes, ctx->stream);
  q->cp.trace = trace_dev;
#endif
  cudaError_t err;
  switch (BN) {
    case 16: err = launch_chain<16, 6, 4>(ctx, *q, grid); break;    // TMEM: 2 x 48 accumulator columns, weights from 128
    case 32: err = launch_chain<32, 5, 4>(ctx, *q, grid); break;    //       2 x 96, weights from 192
    default: err = launch_chain<64, 2, 3>(ctx, *q, grid); break;    //       2 x 192, weights from 384
  }
  if (err != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "projection chain launch (%d phases) failed: %s", n, cudaGetErrorString(err));
  ctx->launches++;
#ifdef PI_CHAIN_TRACE
  if (const char* path = getenv("PI_CHAIN_TRACE_FILE")) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(ctx->stream, &cap);
    if (cap == cudaStreamCaptureStatusNone) {
      std::vector<unsigned long long> host((size_t)256 * 64);
      cudaStreamSynchronize(ctx->stream);
      cudaMemcpy(host.data(), trace_dev, trace_bytes, cudaMemcpyDeviceToHost);
      if (FILE* f = fopen(path, "ab")) {
        const int hdr[4] = {n, grid, BN, 0};
        fwrite(hdr, sizeof(int), 4, f);
        fwrite(host.data(), sizeof(unsigned long long), host.size(), f);
        fclose(f);
      }
    }
  }
#endif
  return PI_OK;
}

pi_status pi_gemm_chain_close(pi_ctx* ctx) {
  ChainQueue* q = static_cast<ChainQueue*>(ctx->gemm_chain);
  if (q) q->open = false;
  return pi_gemm_chain_flush(ctx);
}

// After a bounded wait ran out the barrier words and tickets may be left mid-count: clear them (stream ordered).
void pi_gemm_chain_reset_sync(pi_ctx* ctx) {
  ChainQueue* q = static_cast<ChainQueue*>(ctx->gemm_chain);
  if (!q || !q->ws) return;
  unsigned char* words = static_cast<unsigned char*>(q->ws) + q->ws_slots * (size_t)q->ws_bn * kBM * sizeof(float);
  cudaMemsetAsync(words, 0, (4 * q->ws_tiles + 32 * kMaxPhases) * sizeof(unsigned int), ctx->stream);
}

void pi_gemm_chain_destroy(pi_ctx* ctx) {
  ChainQueue* q = static_cast<ChainQueue*>(ctx->gemm_chain);
  if (!q) return;
  if (q->ws) cudaFree(q->ws);
  delete q;
  ctx->gemm_chain = nullptr;
}

pi_status pi_gemm_chain_enqueue(pi_ctx* ctx, const pi_linear* lin, const pi_linear_args& a, const pi_act_planes& in) {
  ChainQueue* q = queue_of(ctx);
  if (!q) return pi_fail(ctx, PI_ERR_OOM, "host allocation failed");
  const int BN = pi_tc::pick_bn(a.M);
  if (q->n > 0 && (q->n == kMaxPhases || q->BN != BN || q->cp.ph[0].M != a.M)) PI_TRY(pi_gemm_chain_flush(ctx));
  GemmParams p;
  CUtensorMap map;
  PI_TRY(pi_tc::build_gemm_params(ctx, lin, a, in, BN, &p, &map));
  p.ksplit = 1;
  q->cp.ph[q->n] = p;
  q->maps.m[q->n] = map;
  q->cp.rtiles[q->n] = (p.N + kBM - 1) / kBM;
  q->BN = BN;
  ++q->n;
  if (!q->open) return pi_gemm_chain_flush(ctx);
  return PI_OK;
}
