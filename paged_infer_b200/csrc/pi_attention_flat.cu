// Paged-attention decode over a flat work list (block size 16, head_dim 64 / 128).
//
// A batch of ragged windows is a list of K|V tiles: (entry, logical block, kv head).  One launch of the per-entry
// kernel gives every (kv head, entry, KV split) its own short-lived CTA, so short windows leave CTAs nearly empty,
// long ones set the tail, and every warp pays the latency of its first tiles for a handful of tiles of work.
// Here the blocks of the whole batch are laid end to end - entry after entry - and cut into one equal range per
// GROUP of num_kv_heads resident warps; the warps of a group walk the same blocks, one kv head each, so the tiles
// they fetch at about the same time are adjacent in the pool:
//
//   attn_plan_kernel   one CTA, once per step (the positions live on the device and move with every step): window
//                      sizes -> prefix sums -> for every group the SEGMENTS of its range (a segment is the part of
//                      one entry's window that falls into the range), for every warp slot a 64-byte start record
//                      (its segments, the first one's blocks and physical blocks), and for every (entry, kv head)
//                      where its partial results will be and how many there are.
//   attn_decode_flat_kernel   a persistent grid (as many CTAs as fit the GPU at once).  A warp streams the items of its
//                      range - the query rows of a segment, then its K|V tiles - through one ring of bulk copies that
//                      never drains between segments.  The arithmetic per tile is that of attn_decode_v3_kernel.  A
//                      segment that covers its whole window writes the output itself; otherwise it leaves a partial
//                      (m, l, acc) and counts itself in, and the warp that completes the count merges the partials in
//                      slot order - so the sum does not depend on which warp came last - and writes the output (and,
//                      on request, its three bf16 planes for the projection that follows).  No merge launch.
//                      A warp checks what it reads from the work list (segment counts, entry, block range, physical
//                      block) before it reads anything THROUGH it; an inconsistent list ends the step with an error
//                      that names what was found, not with a wild address.
//
// Replaces PagedAttention::run / for_each_block (reference src/attention.rs:141-295) for batched decode.
#include <algorithm>

#include "pi_common.cuh"
#include "pi_attention.cuh"

namespace {

constexpr int kFlatWarps = 4;            // warps per CTA, each with its own ring
constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxB = kPlanThreads;  // one entry per planning thread
constexpr int kPlanMaxWarps = 2 * kPlanThreads;
constexpr int kMinTilesPerWarp = 4;      // shorter ranges are not worth a warp's start-up
constexpr int kSegCap = 8;               // segment descriptors a warp keeps in shared memory (more: read from global)

struct PlanParams {
  const int32_t* lens;
  const int32_t* pos;
  const int32_t* start;
  const int32_t* safe_lb;   // [B] or null
  const int32_t* tables;
  int max_blocks;
  int B, KVH, BS, W;
  int4* hdr;       // [W][4]: everything a warp needs to start its copies, in one 64-byte record (see FlatHeader)
  int4* segs;      // two per group segment: {entry, -, first block, end block}, {position, window start, -, -}
  int2* comb;      // [B * KVH]: {first group segment, number of group segments}; partial slot = segment * KVH + kv head
  int* counters;   // [B * KVH]
};

// hdr[w]: {first segment, end segment, blocks of the first segment that may be fetched before the dependency wait, -}
//         {entry, kv head, first block, end block} and {position, window start, -, -} of the first segment
//         {physical block of its first, second, third tile (or -1), -}
constexpr int kHdrWords = 4;

struct PlanShared {
  int n[kPlanMaxB], first[kPlanMaxB], P[kPlanMaxB + 1], pos[kPlanMaxB], st[kPlanMaxB];
  int so[kPlanMaxWarps + 1];
  int wt[32];
  int total;
};

// Inclusive scan of one value per thread over the CTA (1024 threads); `wt` is scratch for the warp totals.
__device__ __forceinline__ int plan_scan_inclusive(int v, int* wt) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  __syncthreads();   // wt may still be read from an earlier scan
  if (lane == 31) wt[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = wt[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    wt[lane] = w;
  }
  __syncthreads();
  return v + (warp > 0 ? wt[warp - 1] : 0);
}

// Segments of warp group g (the KVH warps that walk one range of blocks, one kv head each): counted, or (EMIT)
// written from group-segment `seg_base` on.
template <bool EMIT>
__device__ int plan_walk(const PlanParams& pp, const PlanShared& s, int r, long T, int g, int seg_base) {
  long t = (long)g * r;
  if (t >= T) return 0;
  const long t1 = min(T, t + (long)r);
  // the entry that holds block t of the list: the first i in [1, B] with P[i] > t, minus one (P[B] = T > t)
  int lo = 1, hi = pp.B;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if ((long)s.P[mid] > t) hi = mid; else lo = mid + 1;
  }
  int b = lo - 1, nb = s.n[b];
  int lbr = (int)(t - (long)s.P[b]);
  int cnt = 0;
  while (t < t1) {
    const int take = (int)min((long)(nb - lbr), t1 - t);
    if (EMIT) {
      const int j = seg_base + cnt, lb0 = s.first[b] + lbr;
      pp.segs[2 * j] = make_int4(b, 0, lb0, lb0 + take);
      pp.segs[2 * j + 1] = make_int4(s.pos[b], s.st[b], 0, 0);
      if (lbr == 0) {   // the segment that opens this entry: its partials are the group segments from here on
        const long off = (long)s.P[b];
        const int2 c = make_int2(j, (int)((off + nb - 1) / r - off / r + 1));
        for (int kvh = 0; kvh < pp.KVH; ++kvh) pp.comb[b * pp.KVH + kvh] = c;
      }
    }
    ++cnt;
    t += take;
    lbr += take;
    if (lbr == nb) {
      lbr = 0;
      do ++b; while (b < pp.B && s.n[b] == 0);
      nb = b < pp.B ? s.n[b] : 1;
    }
  }
  return cnt;
}

__global__ void __launch_bounds__(kPlanThreads) attn_plan_kernel(const PlanParams pp) {
  __shared__ PlanShared s;
  pi_grid_dependency_wait();   // the positions are advanced on the device at the end of a step
  const int tid = threadIdx.x;
  {
    int n = 0, first = 0, pos = 0, st = 0;
    if (tid < pp.B) {
      pos = pp.pos[tid];
      st = pp.start[tid];
      if (st <= pos) {
        first = st / pp.BS;
        n = max(min(pos / pp.BS + 1, pp.lens[tid]) - first, 0);   // blocks past the mapped length are never read
      }
    }
    s.n[tid] = n; s.first[tid] = first; s.pos[tid] = pos; s.st[tid] = st;
    const int inc = plan_scan_inclusive(n, s.wt);
    s.P[tid] = inc - n;
    if (tid == kPlanThreads - 1) s.P[kPlanMaxB] = inc;
  }
  for (int pr = tid; pr < pp.B * pp.KVH; pr += kPlanThreads) {
    pp.comb[pr] = make_int2(0, 0);
    pp.counters[pr] = 0;
  }
  __syncthreads();
  // The list is cut over GROUPS of KVH warp slots: the warps of a group walk the same blocks, one kv head each, so
  // the K|V tiles they fetch at about the same time are the adjacent tiles of one physical block.
  const int NG = pp.W / pp.KVH;
  const long T = (long)s.P[kPlanMaxB];
  const int r = (int)max((T + NG - 1) / NG, (long)kMinTilesPerWarp);
  // two groups per thread, consecutive, so that one scan value per thread orders all segments
  const int g0 = 2 * tid, g1 = 2 * tid + 1;
  const int c0 = g0 < NG ? plan_walk<false>(pp, s, r, T, g0, 0) : 0;
  const int c1 = g1 < NG ? plan_walk<false>(pp, s, r, T, g1, 0) : 0;
  const int inc = plan_scan_inclusive(c0 + c1, s.wt);
  const int base0 = inc - c0 - c1, base1 = base0 + c0;
  if (c0) plan_walk<true>(pp, s, r, T, g0, base0);
  if (c1) plan_walk<true>(pp, s, r, T, g1, base1);
  // the start records of the group's warp slots (this thread wrote the segments it copies from)
  for (int k = 0; k < 2; ++k) {
    const int g = k ? g1 : g0, c = k ? c1 : c0, base = k ? base1 : base0;
    if (g >= NG) continue;
    int4 a = make_int4(0, 0, 0, 0), bq = a, pbs = make_int4(-1, -1, -1, 0);
    int safe = 0;
    if (c) {
      a = pp.segs[2 * base];
      bq = pp.segs[2 * base + 1];
      if ((unsigned)a.x < (unsigned)pp.B && a.z >= 0 && a.z < a.w && a.w <= pp.max_blocks) {
        const int32_t* row = pp.tables + (size_t)a.x * pp.max_blocks;
        pbs.x = row[a.z];
        if (a.z + 1 < a.w) pbs.y = row[a.z + 1];
        if (a.z + 2 < a.w) pbs.z = row[a.z + 2];
        if (pp.safe_lb) safe = pp.safe_lb[a.x];
      }
    }
    for (int kvh = 0; kvh < pp.KVH; ++kvh) {
      const int w = g * pp.KVH + kvh;
      pp.hdr[kHdrWords * w + 0] = make_int4(base, base + c, safe, 0);
      pp.hdr[kHdrWords * w + 1] = make_int4(a.x, kvh, a.z, a.w);
      pp.hdr[kHdrWords * w + 2] = bq;
      pp.hdr[kHdrWords * w + 3] = pbs;
    }
  }
  // warp slots past the last whole group (W not a multiple of KVH) have nothing to do
  for (int w = NG * pp.KVH + tid; w < pp.W; w += kPlanThreads) pp.hdr[kHdrWords * w] = make_int4(0, 0, 0, 0);
}

struct FlatParams {
  const float* q;
  size_t q_stride;
  float* out;
  size_t out_stride;
  const float* kv;
  pi_kv_layout L;
  int layer;
  int B;
  const int32_t* tables;
  int max_blocks;
  const int4* hdr;
  const int4* segs;
  const int2* comb;
  int* counters;
  int plan_settled;  // the work list was complete before the kernel ahead of this one started: it may be read early
  int max_slots;     // segments (= partial slots) the work list has room for
  float* part_acc;   // [slot][G][HD]
  float* part_ml;    // [slot][G][2]   (running max in the log2 domain, sum)
  float scale;
  int* err_flag;
  unsigned short* emit_base;   // output as three bf16 planes [3][.][emit_k] as well, or null
  size_t emit_plane_stride;
  int emit_k;
};

// A warp that finds its part of the work list inconsistent (a segment count, an entry, a block range or a physical
// block outside the batch) reads nothing through it: it records what it saw once, raises the error word and stops.
__device__ __noinline__ void flat_report(int* err, int code, int wslot, int s0, int s1, int4 seg, int pb, int item) {
  if (!err) return;
  if (atomicCAS(err + 1, 0, code) == 0) {
    err[2] = wslot; err[3] = s0; err[4] = s1;
    err[5] = seg.x; err[6] = seg.y; err[7] = seg.z; err[8] = seg.w;
    err[9] = pb; err[10] = item;
    __threadfence();
  }
  atomicExch(err, code);
}

// Four consecutive outputs of (entry b, head h) from dim d: the f32 row and, on request, its planes.
__device__ __forceinline__ void flat_store4(const FlatParams& p, int b, int h, int HD, int d, float4 v) {
  *reinterpret_cast<float4*>(p.out + (size_t)b * p.out_stride + (size_t)h * HD + d) = v;
  if (p.emit_base) {
    const float y[4] = {v.x, v.y, v.z, v.w};
    unsigned short a[4], bb[4], c[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) pi_split3(y[j], a[j], bb[j], c[j]);
    unsigned short* base = p.emit_base + (size_t)b * p.emit_k + (size_t)h * HD + d;
    *reinterpret_cast<uint2*>(base) = make_uint2((uint32_t)a[0] | ((uint32_t)a[1] << 16), (uint32_t)a[2] | ((uint32_t)a[3] << 16));
    *reinterpret_cast<uint2*>(base + p.emit_plane_stride) =
        make_uint2((uint32_t)bb[0] | ((uint32_t)bb[1] << 16), (uint32_t)bb[2] | ((uint32_t)bb[3] << 16));
    *reinterpret_cast<uint2*>(base + 2 * p.emit_plane_stride) =
        make_uint2((uint32_t)c[0] | ((uint32_t)c[1] << 16), (uint32_t)c[2] | ((uint32_t)c[3] << 16));
  }
}

template <int HD, int G, int STAGES>
__global__ void __launch_bounds__(kFlatWarps * 32) attn_decode_flat_kernel(const FlatParams p) {
  constexpr int BS = 16;
  constexpr int LPT = HD / 8;       // lanes per token
  constexpr int TPW = 32 / LPT;     // tokens per warp step
  constexpr int STEPS = BS / TPW;   // steps per tile
  constexpr uint32_t kTileBytes = 2u * BS * HD * sizeof(float);
  constexpr uint32_t kQBytes = (uint32_t)(G * HD * sizeof(float));
  constexpr float kLog2e = 1.4426950408889634f;
  static_assert(kQBytes <= kTileBytes, "the query rows of a segment travel through a tile slot");
  extern __shared__ __align__(128) unsigned char flat_smem[];
  __shared__ __align__(8) unsigned long long bars[kFlatWarps][STAGES];
  __shared__ int4 s_segs[kFlatWarps][2 * kSegCap];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tg = lane / LPT, li = lane % LPT;
  const int wslot = blockIdx.x * kFlatWarps + warp, W = gridDim.x * kFlatWarps;
  const int KVH = p.L.num_kv_heads;
  const int my_kvh = wslot % KVH;   // the warps of a group walk the same blocks, one kv head each
  float* ring = reinterpret_cast<float*>(flat_smem) + (size_t)warp * STAGES * (kTileBytes / 4);

  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(attn_smem_u32(&bars[warp][s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  // ---- the copies: item after item of the range, STAGES ahead of the arithmetic ---------------------------------
  // Item order: for every segment its query rows, then its tiles.  Every lane tracks the position (cheap and
  // uniform); lane 0 looks up the physical block of the NEXT tile right after a copy goes out, so the table read is
  // never on the path between two tiles.  The first tiles' physical blocks come with the warp's start record.
  int s0 = 0, s1 = 0, is = 0, ji = 0, ilb = 0, pb_next = -1, first_lb0 = 0;
  int4 ia = make_int4(0, 0, 0, 0), hpb = make_int4(-1, -1, -1, 0);
  bool iq = true, bad = false;
  uint32_t pre_issued = 0;   // items whose copy went out before the dependency wait
  auto seg_ok = [&](const int4& sg) {
    return (unsigned)sg.x < (unsigned)p.B && (unsigned)sg.y < (unsigned)KVH && sg.z >= 0 && sg.z < sg.w && sg.w <= p.max_blocks;
  };
  auto copy_tile = [&](int item, int kvh, int pb) {   // lane 0
    const uint32_t bar = attn_smem_u32(&bars[warp][item % STAGES]);
    const uint32_t dst = attn_smem_u32(ring + (size_t)(item % STAGES) * (kTileBytes / 4));
    const float* src = p.kv + pi_kv_tile_offset(p.L, p.layer, pb, kvh, 0);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kTileBytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(kTileBytes), "r"(bar)
                 : "memory");
  };
  auto hdr_pb = [&](int k) { return k == 0 ? hpb.x : (k == 1 ? hpb.y : hpb.z); };
  auto read_header = [&]() {
    const int4 h0 = p.hdr[kHdrWords * wslot];
    s0 = h0.x;
    s1 = h0.y;
    if (s0 < 0 || s1 < s0 || s1 * KVH > p.max_slots) {
      if (lane == 0) flat_report(p.err_flag, 11, wslot, s0, s1, make_int4(0, 0, 0, 0), -1, -1);
      s0 = s1 = 0;
      bad = true;
    }
    if (s0 < s1) {
      ia = p.hdr[kHdrWords * wslot + 1];
      hpb = p.hdr[kHdrWords * wslot + 3];
    }
    return h0.z;
  };
  bool have_header = false;
  if (p.plan_settled) {
    // Tiles of blocks that were complete when the batch was uploaded do not depend on the kernel ahead of this one:
    // the first tiles of the ring go out before the dependency wait (items 1.. ; item 0 is the query rows).
    const int safe = read_header();
    have_header = true;
    if (lane == 0 && s0 < s1 && seg_ok(ia))
      for (int k = 0; k + 1 < STAGES && ia.z + k < min(ia.w, safe) && (unsigned)hdr_pb(k) < (unsigned)p.L.num_blocks; ++k) {
        copy_tile(k + 1, ia.y, hdr_pb(k));
        pre_issued |= 1u << (k + 1);
      }
    pre_issued = __shfl_sync(0xffffffffu, pre_issued, 0);
  }
  pi_grid_dependency_wait();   // the work list (unless settled), the query rows and this step's K/V rows come from kernels ahead
  if (!have_header) read_header();
  is = s0;   // a slot without segments (s0 == s1) issues nothing
  if (s0 < s1) {
    ilb = ia.z;
    first_lb0 = ia.z;
    pb_next = hpb.x;
  }
  bool cache_ready = false;   // s_segs holds this warp's first segments
  auto seg_word = [&](int s, int half) -> int4 {
    int4 v = (cache_ready && s - s0 < kSegCap) ? s_segs[warp][2 * (s - s0) + half] : __ldg(&p.segs[2 * s + half]);
    if (half == 0) v.y = my_kvh;   // the list is shared by the group's warps
    return v;
  };
  auto issue_one = [&]() {
    const uint32_t bar = attn_smem_u32(&bars[warp][ji % STAGES]);
    const uint32_t dst = attn_smem_u32(ring + (size_t)(ji % STAGES) * (kTileBytes / 4));
    if (iq) {
      if (!seg_ok(ia)) {
        if (lane == 0) flat_report(p.err_flag, 12, wslot, s0, s1, ia, -1, ji);
        bad = true;
        is = s1;   // nothing further goes out
        return;
      }
      if (lane == 0) {
        const float* src = p.q + (size_t)ia.x * p.q_stride + (size_t)ia.y * G * HD;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kQBytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                     "r"(kQBytes), "r"(bar)
                     : "memory");
      }
      iq = false;
    } else {
      const int pbv = __shfl_sync(0xffffffffu, pb_next, 0);
      if ((unsigned)pbv >= (unsigned)p.L.num_blocks) {
        if (lane == 0) flat_report(p.err_flag, 13, wslot, s0, s1, ia, pbv, ji);
        bad = true;
        is = s1;
        return;
      }
      if (lane == 0 && !(ji < STAGES && ((pre_issued >> ji) & 1u))) copy_tile(ji, ia.y, pbv);
      if (++ilb >= ia.w) {
        if (++is < s1) {
          ia = seg_word(is, 0);
          ilb = ia.z;
          iq = true;
        }
      }
      if (lane == 0 && is < s1)
        pb_next = (is == s0 && ilb - first_lb0 < 3) ? hdr_pb(ilb - first_lb0)
                  : (seg_ok(ia) && ilb < ia.w)      ? p.tables[(size_t)ia.x * p.max_blocks + ilb]
                                                    : -1;   // reported when the copy is due
    }
    ++ji;
  };
  // wait for item j of this warp; false when the bounded wait ran out
  auto wait_item = [&](int j) -> bool {
    const uint32_t bar = attn_smem_u32(&bars[warp][j % STAGES]);
    const uint32_t parity = (j / STAGES) & 1;
    uint32_t done = 0;
    for (uint32_t spin = 0; spin < kAttnSpinLimit && !done; ++spin)
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return __all_sync(0xffffffffu, done != 0);
  };
#pragma unroll 1
  while (ji < STAGES && is < s1) issue_one();   // (a first segment shorter than the ring reads the next one's words from global memory)
  // an (entry, kv head) with an empty window has no segment: its output rows are zeros
  for (int pr = wslot; pr < p.B * KVH; pr += W) {
    if (p.comb[pr].y != 0) continue;
    const int b = pr / KVH, kvh = pr - b * KVH;
    for (int idx = lane; idx < G * HD / 4; idx += 32)
      flat_store4(p, b, kvh * G + idx / (HD / 4), HD, (idx % (HD / 4)) * 4, make_float4(0.f, 0.f, 0.f, 0.f));
  }
  if (s0 >= s1) return;
  if (lane < 2 * min(s1 - s0, kSegCap)) s_segs[warp][lane] = p.segs[2 * s0 + lane];
  __syncwarp();
  cache_ready = true;

  const float scale2 = p.scale * kLog2e;
  const int lane_base = lane & ~(LPT - 1);
  int jc = 0;
  bool failed = false;

#pragma unroll 1
  for (int cs = s0; cs < s1; ++cs) {
    const int4 sa = seg_word(cs, 0), sb = seg_word(cs, 1);
    const int b = sa.x, kvh = sa.y, lb0 = sa.z, lb1 = sa.w, pos = sb.x, st = sb.y;
    if (!seg_ok(sa)) {
      if (lane == 0) flat_report(p.err_flag, 12, wslot, s0, s1, sa, -1, -2);
      failed = bad = true;
      break;
    }
    const int2 cm = __ldg(&p.comb[b * KVH + kvh]);   // needed at the end of the segment only

    // ---- the query rows: 8 dims per lane (16-byte chunks li and li + LPT of the head) for every head of the group
    if (jc >= ji || !wait_item(jc)) { failed = true; break; }
    float2 qv[G][4];
    {
      const float* qs = ring + (size_t)(jc % STAGES) * (kTileBytes / 4);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float4 a = *reinterpret_cast<const float4*>(qs + g * HD + li * 4);
        const float4 c = *reinterpret_cast<const float4*>(qs + g * HD + (li + LPT) * 4);
        qv[g][0] = make_float2(a.x, a.y); qv[g][1] = make_float2(a.z, a.w);
        qv[g][2] = make_float2(c.x, c.y); qv[g][3] = make_float2(c.z, c.w);
      }
    }
    __syncwarp();
    if (is < s1) issue_one();
    ++jc;

    float2 acc[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[g][i] = make_float2(0.f, 0.f);
    // softmax state of the head this lane owns (log2 domain), over the tokens of its token group
    float m_own = -INFINITY, l_own = 0.f;

#pragma unroll 1
    for (int lb = lb0; lb < lb1; ++lb) {
      if (jc >= ji || !wait_item(jc)) { failed = true; break; }
      const int t_lo = max(st - lb * BS, 0), t_hi = min(pos - lb * BS, BS - 1);
      const bool whole = (t_lo == 0) && (t_hi == BS - 1);
      const float* Kt = ring + (size_t)(jc % STAGES) * (kTileBytes / 4);
      const float* Vt = Kt + BS * HD;

      // ---- A: scores -----------------------------------------------------------------------------------------
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
      if (is < s1) issue_one();
      ++jc;
    }
    if (failed) break;

    // ---- end of the segment: merge the token groups of the warp (the owned head's m, l; every head's accumulator)
    float m_all = m_own;
#pragma unroll
    for (int o = LPT; o < 32; o <<= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
    const float f_own = (m_own == -INFINITY) ? 0.f : ex2_approx(m_own - m_all);
    float l_all = l_own * f_own;
#pragma unroll
    for (int o = LPT; o < 32; o <<= 1) l_all += __shfl_xor_sync(0xffffffffu, l_all, o);
    if (cm.y < 1 || cm.x < 0 || (cm.x + cm.y) * KVH > p.max_slots || cs < cm.x || cs >= cm.x + cm.y) {
      if (lane == 0) flat_report(p.err_flag, 12, wslot, s0, s1, make_int4(b, kvh, cm.x, cm.y), -1, -3);
      failed = bad = true;
      break;
    }
    const bool direct = cm.y == 1;   // this segment is the whole window: normalise and write the output rows
    const float inv_own = 1.0f / fmaxf(l_all, 1e-12f);
    const int slot = cs * KVH + kvh; // a partial's slot: (group segment, kv head)
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int src_lane = lane_base + attn_owner_lane<G, LPT>(g);
      const float fg = __shfl_sync(0xffffffffu, f_own, src_lane);
      const float ig = __shfl_sync(0xffffffffu, inv_own, src_lane);
      const float2 f2 = make_float2(fg, fg);
      float2 a[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = __fmul2_rn(acc[g][i], f2);
#pragma unroll
        for (int o = LPT; o < 32; o <<= 1) {
          a[i].x += __shfl_xor_sync(0xffffffffu, a[i].x, o);
          a[i].y += __shfl_xor_sync(0xffffffffu, a[i].y, o);
        }
      }
      if (g % TPW == tg) {   // every token group holds the sums now: the groups share the stores
        if (direct) {
          flat_store4(p, b, kvh * G + g, HD, li * 4, make_float4(a[0].x * ig, a[0].y * ig, a[1].x * ig, a[1].y * ig));
          flat_store4(p, b, kvh * G + g, HD, (li + LPT) * 4, make_float4(a[2].x * ig, a[2].y * ig, a[3].x * ig, a[3].y * ig));
        } else {
          float* dstp = p.part_acc + ((size_t)slot * G + g) * HD;
          *reinterpret_cast<float4*>(dstp + li * 4) = make_float4(a[0].x, a[0].y, a[1].x, a[1].y);
          *reinterpret_cast<float4*>(dstp + (li + LPT) * 4) = make_float4(a[2].x, a[2].y, a[3].x, a[3].y);
        }
      }
    }
    if (!direct) {
      const int g_own = attn_owned_head<G, LPT>(li);
      if (tg == 0 && attn_owner_lane<G, LPT>(g_own) == li)   // one writer per head
        *reinterpret_cast<float2*>(p.part_ml + ((size_t)slot * G + g_own) * 2) = make_float2(m_all, l_all);
      __threadfence();
      __syncwarp();
      int old = 0;
      if (lane == 0) old = atomicAdd(&p.counters[b * KVH + kvh], 1);
      old = __shfl_sync(0xffffffffu, old, 0);
      if (old == cm.y - 1) {
        // the last of this (entry, kv head)'s segments to finish merges all of them, in slot order
        __threadfence();
        if (lane == 0) p.counters[b * KVH + kvh] = 0;   // everyone has counted: ready for the next launch
        const int first = cm.x, cnt = cm.y;
        // lane = (head, quarter of its dims): one pass over the partials' (m, l), then all accumulator loads of a
        // group of partials in flight at once
        constexpr int LH = (32 / G < HD / 4) ? 32 / G : HD / 4;   // lanes per head
        constexpr int IPL = (HD / 4) / LH;                         // float4 items per lane
        constexpr int U = IPL > 4 ? 2 : 4;                         // partials in flight at once
        const int g = min(lane / LH, G - 1), dq = lane % LH;
        const bool active = lane / LH < G;
        float M = -INFINITY;
        for (int i = 0; i < cnt; ++i) M = fmaxf(M, __ldcg(p.part_ml + ((size_t)((first + i) * KVH + kvh) * G + g) * 2));
        float ls = 0.f;
        float4 av[IPL];
#pragma unroll
        for (int it = 0; it < IPL; ++it) av[it] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int i0 = 0; i0 < cnt; i0 += U) {
          float2 ml[U];
          float4 pa[U][IPL];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int i = min(i0 + u, cnt - 1);
            const size_t sl = (size_t)(first + i) * KVH + kvh;
            ml[u] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (sl * G + g) * 2));
#pragma unroll
            for (int it = 0; it < IPL; ++it)
              pa[u][it] = __ldcg(reinterpret_cast<const float4*>(p.part_acc + (sl * G + g) * HD + (dq + it * LH) * 4));
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (i0 + u >= cnt) break;
            const float f = (ml[u].x == -INFINITY) ? 0.f : ex2_approx(ml[u].x - M);
            ls += ml[u].y * f;
#pragma unroll
            for (int it = 0; it < IPL; ++it) {
              av[it].x += pa[u][it].x * f; av[it].y += pa[u][it].y * f; av[it].z += pa[u][it].z * f; av[it].w += pa[u][it].w * f;
            }
          }
        }
        const float inv = 1.0f / fmaxf(ls, 1e-12f);
#pragma unroll
        for (int it = 0; it < IPL; ++it)
          if (active)
            flat_store4(p, b, kvh * G + g, HD, (dq + it * LH) * 4,
                      make_float4(av[it].x * inv, av[it].y * inv, av[it].z * inv, av[it].w * inv));
      }
    }
  }

  if (failed) {
    if (lane == 0 && p.err_flag && !bad) atomicExch(p.err_flag, 7);
    for (int jj = jc; jj < ji; ++jj) wait_item(jj);   // bounded drain of the copies still in flight
  }
}

template <int HD, int G, int STAGES>
cudaError_t launch_flat_one(pi_ctx* ctx, int ctas, const FlatParams& p, size_t smem, int* ctas_per_sm) {
  auto k = attn_decode_flat_kernel<HD, G, STAGES>;
  static pi_smem_grant granted;
  static int occupancy[64] = {};
  if (smem > granted.of(ctx)) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    granted.of(ctx) = smem;
    occupancy[(unsigned)ctx->device & 63u] = 0;
  }
  int& occ = occupancy[(unsigned)ctx->device & 63u];
  if (occ == 0) {
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k, kFlatWarps * 32, smem);
    if (e != cudaSuccess) return e;
    if (occ < 1) occ = 1;
  }
  if (ctas_per_sm) {   // a query: how many CTAs of this kernel are resident at once
    *ctas_per_sm = occ;
    return cudaSuccess;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(kFlatWarps * 32);
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
cudaError_t launch_flat(pi_ctx* ctx, int group, int ctas, const FlatParams& p, size_t smem, int* ctas_per_sm) {
  switch (group) {
    case 1: return launch_flat_one<HD, 1, STAGES>(ctx, ctas, p, smem, ctas_per_sm);
    case 2: return launch_flat_one<HD, 2, STAGES>(ctx, ctas, p, smem, ctas_per_sm);
    case 4: return launch_flat_one<HD, 4, STAGES>(ctx, ctas, p, smem, ctas_per_sm);
    default: return launch_flat_one<HD, 8, STAGES>(ctx, ctas, p, smem, ctas_per_sm);
  }
}

size_t flat_ring_bytes(int HD) {
  const size_t tile_bytes = 2 * (size_t)16 * HD * sizeof(float);
  return (size_t)kFlatWarps * (HD == 64 ? 3 : 2) * tile_bytes;
}

cudaError_t flat_dispatch(pi_ctx* ctx, int HD, int group, int ctas, const FlatParams& p, int* ctas_per_sm) {
  return HD == 64 ? launch_flat<64, 3>(ctx, group, ctas, p, flat_ring_bytes(64), ctas_per_sm)
                  : launch_flat<128, 2>(ctx, group, ctas, p, flat_ring_bytes(128), ctas_per_sm);
}

}  // namespace

// Decides whether the batch goes over the flat work list and, if so, queues the kernel that builds the list from the
// positions as they are on the device at that point of the stream.  Call once per step, before the first layer.
pi_status pi_attention_prepare(pi_ctx* ctx, const pi_kv_pool* pool, int num_heads, const pi_attn_batch& batch) {
  batch.flat_warps = 0;
  const pi_kv_layout& L = pool->L;
  if (!ctx->opt_attn_flat || ctx->opt_attn_tma != 1 || L.block_size != 16) return PI_OK;
  if (L.num_kv_heads <= 0 || num_heads <= 0 || num_heads % L.num_kv_heads != 0) return PI_OK;
  const int group = num_heads / L.num_kv_heads, HD = L.head_dim, KVH = L.num_kv_heads;
  if (!(HD == 64 || HD == 128) || !(group == 1 || group == 2 || group == 4 || group == 8)) return PI_OK;
  if (batch.B > kPlanMaxB || (batch.shared_table && batch.B > 1)) return PI_OK;
  if (flat_ring_bytes(HD) + 4096 > ctx->smem_optin) return PI_OK;
  int per_sm = 0;
  FlatParams none = {};
  cudaError_t e = flat_dispatch(ctx, HD, group, 0, none, &per_sm);
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "attention occupancy query failed: %s", cudaGetErrorString(e));
  const int W = std::min(ctx->sm_count * per_sm * kFlatWarps, kPlanMaxWarps) / kFlatWarps * kFlatWarps;
  // few tiles: the per-entry grid starts as many warps and needs no plan
  if (batch.total_window_blocks * KVH < (long)W * kMinTilesPerWarp) return PI_OK;

  const size_t pairs = (size_t)batch.B * KVH, slots = (size_t)W + pairs;
  const size_t off_segs = (size_t)W * kHdrWords * sizeof(int4);
  const size_t off_comb = off_segs + 2 * slots * sizeof(int4);
  const size_t off_cnt = off_comb + pairs * sizeof(int2);
  PI_TRY(pi_reserve(ctx, &ctx->attn_plan, off_cnt + pairs * sizeof(int)));
  PI_TRY(pi_reserve(ctx, &ctx->attn_partial, slots * (size_t)group * (HD + 2) * sizeof(float)));
  unsigned char* base = static_cast<unsigned char*>(ctx->attn_plan.ptr);
  PlanParams pp;
  pp.lens = batch.lens;
  pp.pos = batch.pos;
  pp.start = batch.start;
  pp.B = batch.B;
  pp.KVH = KVH;
  pp.BS = L.block_size;
  pp.W = W;
  pp.safe_lb = batch.safe_lb;
  pp.tables = batch.tables;
  pp.max_blocks = batch.max_blocks;
  pp.hdr = reinterpret_cast<int4*>(base);
  pp.segs = reinterpret_cast<int4*>(base + off_segs);
  pp.comb = reinterpret_cast<int2*>(base + off_comb);
  pp.counters = reinterpret_cast<int*>(base + off_cnt);
  pi_prof_scope prof(ctx, PI_PROF_ATTENTION);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(kPlanThreads);
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, attn_plan_kernel, pp);
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "attention plan launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  batch.flat_warps = W;
  batch.flat_slots = slots;
  batch.flat_hdr = pp.hdr;
  batch.flat_settled = false;
  batch.flat_segs = pp.segs;
  batch.flat_comb = pp.comb;
  batch.flat_counters = pp.counters;
  return PI_OK;
}

// The decode launch over a prepared work list (see pi_attention_prepare); the caller has checked the shape.
pi_status pi_launch_attention_flat(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads, const float* q,
                                   size_t q_stride, float* out, size_t out_stride, const pi_attn_batch& batch,
                                   pi_act_planes* emit, bool* emitted) {
  const pi_kv_layout& L = pool->L;
  const int group = num_heads / L.num_kv_heads, HD = L.head_dim;
  PI_REQUIRE(ctx, ctx->attn_plan.ptr && batch.flat_hdr == ctx->attn_plan.ptr,
             "the attention work list was replaced since this batch was prepared");
  FlatParams p;
  p.q = q;
  p.q_stride = q_stride;
  p.out = out;
  p.out_stride = out_stride;
  p.kv = pool->data;
  p.L = L;
  p.layer = layer;
  p.B = batch.B;
  p.tables = batch.tables;
  p.max_blocks = batch.max_blocks;
  p.hdr = static_cast<const int4*>(batch.flat_hdr);
  p.plan_settled = batch.flat_settled ? 1 : 0;
  p.max_slots = (int)batch.flat_slots;
  p.segs = static_cast<const int4*>(batch.flat_segs);
  p.comb = static_cast<const int2*>(batch.flat_comb);
  p.counters = batch.flat_counters;
  p.part_acc = static_cast<float*>(ctx->attn_partial.ptr);
  p.part_ml = p.part_acc + batch.flat_slots * (size_t)group * HD;
  p.scale = 1.0f / sqrtf((float)HD);
  p.err_flag = ctx->dev_err;
  p.emit_base = nullptr;
  p.emit_plane_stride = 0;
  p.emit_k = 0;
  if (emit && emit->base && emit->K == num_heads * HD && emit->K % 4 == 0 && emit->plane_stride % 4 == 0) {
    p.emit_base = reinterpret_cast<unsigned short*>(emit->base);
    p.emit_plane_stride = emit->plane_stride;
    p.emit_k = emit->K;
    emit->row_scale = nullptr;
    emit->sumsq_tiles = 0;
    if (emitted) *emitted = true;
  }
  cudaError_t e = flat_dispatch(ctx, HD, group, batch.flat_warps / kFlatWarps, p, nullptr);
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  return PI_OK;
}
