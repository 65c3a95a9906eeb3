#!/usr/bin/env python3
"""Benchmark of the int8 paged-decode hot path on B200.

Default workload (`tinyllama_b64_paged`): TinyLlama-1.1B architecture, random-init
int8 projections (lm_head int8 as well), 64 concurrent sequences with context
lengths uniform in [256, 2048] (seed 2), KV block size 16, f32 KV; sequences
0-31 share the physical blocks of a common 512-token prefix, sequences 56-63
are copy-on-write forks of 48-55; one greedy decode step per sequence per
engine step.  A "step" is one engine step over all 64 sequences.

  value      decode tok/s with everything resident on the device: K greedy steps
             inside one `pi_model_decode_multi` call (no host round trip between
             steps), timed with CUDA events.
  e2e        the same metric through the per-step public call
             (`LlamaWeights.decode_batch_into`): block-table bookkeeping on the
             host, tokens / tables / positions copied host->device and the
             chosen ids device->host inside the timed region, every step.
  roofline   the dominant kernel timed alone with CUDA events.
  cpu_baseline  the CPU oracle (a C++ restatement of the reference's rayon/AVX2
             path; the reference itself is Rust and cannot be built here) on a
             bounded sample of the same workload, on this box's host cores.

`--impl reference` times that CPU path as the reference arm.  With `--gpus N`
under torchrun every rank runs its own replica of the workload (sequences are
independent; no collective on the data path): weak scaling.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BLOCK = 16
TINYLLAMA = dict(hidden_size=2048, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4,
                 intermediate_size=5632, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)
# DRAM traffic (dram__bytes_read + dram__bytes_write of one profiler capture) divided by the algorithmic bytes of the
# same launch, per kernel class, from small single-kernel captures (`--kernel-case`, summaries under profiles/):
# traffic of a bench launch = ratio x its algorithmic bytes (traffic grows in proportion to the rows / tokens streamed).
NCU_TRAFFIC_RATIO = {"gemm_tc": 1.05, "gemv": 1.003, "attention": 1.03}
GEMV_SHAPES = {"q/o 2048x2048": (2048, 2048), "k/v 256x2048": (256, 2048), "qkv fused 2560x2048": (2560, 2048),
               "gate/up 5632x2048": (5632, 2048), "down 2048x5632": (2048, 5632), "lm_head 32000x2048": (32000, 2048),
               "lm_head Llama-3 128256x4096": (128256, 4096)}


# ---- host-side block bookkeeping (what KvCacheManager does for this workload) ---------------------------------
class PagedBatch:
    """Block tables of the 64-sequence workload: a refcounted free list, prefix
    sharing at admission, fork = table copy, copy-on-write before a write into a
    shared block (reference src/memory/allocator.rs, kv_cache_manager.rs:116-345)."""

    def __init__(self, seed: int, batch: int, total_steps: int, lo=256, hi=2048, prefix_tokens=512, forks=8):
        rng = np.random.default_rng(seed)
        self.batch = batch
        ctx = rng.integers(lo, hi + 1, batch)
        if forks:
            ctx[batch - forks:] = ctx[batch - 2 * forks:batch - forks]   # a fork starts at its parent's length
        self.lengths = [int(c) for c in ctx]
        need = sum((c + total_steps + BLOCK - 1) // BLOCK + 1 for c in self.lengths)
        self.num_blocks = need + 8
        self.free = list(range(self.num_blocks))[::-1]
        self.ref = [0] * self.num_blocks
        self.tables = []
        self.cow_copies = []          # (src, dst) pairs produced by the last plan()
        self.total_cow = 0
        shared = []
        for b in range(batch):
            nblk = (self.lengths[b] + BLOCK - 1) // BLOCK
            if forks and b >= batch - forks:               # fork: same table as the parent, refcounts bumped
                t = list(self.tables[b - forks])
                for pb in t:
                    self.ref[pb] += 1
            else:
                t = []
                if b < batch // 2:                          # prefix-cache hit on full blocks only
                    n_shared = min(prefix_tokens // BLOCK, self.lengths[b] // BLOCK)
                    while len(shared) < n_shared:
                        shared.append(self._alloc())
                    for pb in shared[:n_shared]:
                        self.ref[pb] += 1
                        t.append(pb)
                while len(t) < nblk:
                    t.append(self._alloc())
            self.tables.append(t)
        for pb in shared:                                   # the cache's own reference
            self.ref[pb] += 1
        self.packed = None                                  # PackedBlockTables mirror, kept in step by plan()

    def _alloc(self) -> int:
        pb = self.free.pop()
        self.ref[pb] = 1
        return pb

    def plan(self):
        """Before a step: give every sequence a writable slot for position len(seq)."""
        self.cow_copies = []
        for b in range(self.batch):
            pos, t = self.lengths[b], self.tables[b]
            lb = pos // BLOCK
            if lb >= len(t):
                t.append(self._alloc())
                if self.packed is not None:
                    self.packed.append(b, t[-1])
            elif self.ref[t[lb]] > 1:                       # ensure_writable: copy-on-write split
                dst = self._alloc()
                self.cow_copies.append((t[lb], dst))
                self.ref[t[lb]] -= 1
                t[lb] = dst
                if self.packed is not None:
                    self.packed.remap(b, lb, dst)
        self.total_cow += len(self.cow_copies)
        return self.cow_copies

    def commit(self):
        self.lengths = [n + 1 for n in self.lengths]

    def pack(self, api):
        """The tables as arrays, from now on updated in place by plan() (what an engine's FFI shim would keep)."""
        self.packed = api.PackedBlockTables(self.batch, max(len(t) for t in self.tables) + 8)
        for b, t in enumerate(self.tables):
            self.packed.set_row(b, t)
        return self.packed

    def unique_mapped_tokens(self) -> int:
        """Tokens of KV that one step must read at least once (shared physical blocks count once)."""
        seen = {}
        for n, t in zip(self.lengths, self.tables):
            for lb, pb in enumerate(t):
                used = min(BLOCK, n + 1 - lb * BLOCK)
                if used > 0:
                    seen[pb] = max(seen.get(pb, 0), used)
        return sum(seen.values())

    def logical_tokens(self) -> int:
        return sum(n + 1 for n in self.lengths)


# ---- clocks ---------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.rows, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.device)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 9] or [r for _, r in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[1]) for r in rows)
        reasons = set()
        for r in rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][2]), "power_w_max": max(float(r[3]) for r in rows),
                "samples": len(rows), "reasons": sorted(reasons)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- the CPU arm (oracle) ---------------------------------------------------------------------------------------
def cpu_decode_sample(cfg: dict, pb: PagedBatch, budget_s: float, max_steps: int, warmup: int = 1):
    """Time oracle decode steps of the same 64 sequences on the host cores."""
    from oracle import pi_oracle as orc
    orc.build()
    rng = np.random.default_rng(7)
    H, NL, KH = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_key_value_heads"]
    hd = H // cfg["num_attention_heads"]
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]

    def i8(rows, cols):
        return (rng.integers(-127, 128, (rows, cols), dtype=np.int8), np.full(rows, 1.6e-4, np.float32))

    shapes = {"wq": (H, H), "wk": (KH * hd, H), "wv": (KH * hd, H), "wo": (H, H), "w1": (inter, H), "w2": (H, inter), "w3": (inter, H)}
    layer0 = {k: i8(*s) for k, s in shapes.items()}       # timing does not depend on the values: reuse one layer's codes
    projs = [layer0] * NL
    embed = rng.integers(0x3B00, 0x3C00, (vocab, H), dtype=np.uint16)  # small positive bf16 values
    ones = np.ones(H, np.float32)
    model = orc.Model(cfg, embed, ones, [ones] * NL, [ones] * NL, projs, i8(vocab, H))
    layout_floats = NL * pb.num_blocks * BLOCK * KH * 2 * hd
    chunk = rng.standard_normal(1 << 22).astype(np.float32)
    kv = np.resize(chunk, layout_floats)
    tokens = rng.integers(0, vocab, pb.batch).astype(np.uint32)
    times = []
    t_start = time.time()
    for s in range(warmup + max_steps):
        pb.plan()
        t0 = time.perf_counter()
        logits = model.decode_batch(tokens, pb.lengths, pb.tables, kv, BLOCK)
        tokens = np.array([orc.argmax(r) for r in logits], np.uint32)
        dt = time.perf_counter() - t0
        pb.commit()
        if s >= warmup:
            times.append(dt)
        if time.time() - t_start > budget_s and len(times) >= 1:
            break
    return times, orc.num_threads(), orc.backend()


def run_reference_arm(args, rank: int):
    if rank != 0:
        return
    cfg = dict(TINYLLAMA)
    pb = PagedBatch(2, 64, args.steps + args.warmup + 2)
    times, threads, backend = cpu_decode_sample(cfg, pb, budget_s=150.0, max_steps=args.steps, warmup=min(args.warmup, 1))
    ms = 1e3 * float(np.mean(times))
    val = 64.0 / (ms / 1e3)
    sample = (f"{len(times)} of the requested {args.steps} steps (time-bounded), each a full 64-sequence engine step "
              f"(contexts U[256,2048], block 16) on the CPU oracle, {backend}, {threads} threads")
    line = {
        "impl": "reference", "metric": "int8 batched paged decode throughput (TinyLlama-1.1B arch, 64 sequences)",
        "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": len(times), "warmup": min(args.warmup, 1),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 weights, f32 activations/accumulate/KV",
        "data": "synthetic", "config": {"workload": "tinyllama_b64_paged", "batch": 64, "block_size": BLOCK, "context": "U[256,2048] seed 2"},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference is a Rust crate and cannot be built on this box (no cargo/rustc); this arm is its C++ restatement (oracle/)",
    }
    print(json.dumps(line), flush=True)


# ---- the GPU arm ---------------------------------------------------------------------------------------------------
def gemv_sweep(api, ctx, torch, hbm_peak, reps=3):
    """Config-1 style isolated projections at M=1: weight copies rotate so that every launch streams from HBM."""
    out = {}
    rng = np.random.default_rng(1)
    for name, (N, K) in GEMV_SHAPES.items():
        bytes_w = N * K + 4 * N
        copies = int(min(48, max(2, -(-(400 << 20) // bytes_w))))
        q = rng.integers(-127, 128, (N, K), dtype=np.int8)
        s = np.full(N, 1.6e-4, np.float32)
        lins = [api.Projection.int8(ctx, q, s) for _ in range(copies)]
        x = torch.randn(1, K, device="cuda", dtype=torch.float32)
        y = torch.empty(1, N, device="cuda", dtype=torch.float32)
        for l in lins:
            l.apply_device(x, y, 1)
        torch.cuda.synchronize()
        best = None
        for _ in range(reps):
            # back-to-back launches over the rotating copies, one CUDA-event pair around the whole train on the
            # launching stream: per-launch = total / launches (a pair of events per launch would add ~4 us each)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _r in range(4):
                for l in lins:
                    l.apply_device(x, y, 1)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (4 * copies)
            best = us if best is None else min(best, us)
        algo = N * K + 4 * N + 4 * K + 4 * N
        out[name] = {"us": round(best, 3), "GB/s": round(algo / best / 1e3, 1), "frac_of_hbm_peak": round(algo / best / 1e3 / hbm_peak, 3),
                     "bytes": algo, "hbm_resident_rotation": copies * bytes_w > (256 << 20)}
        for l in lins:
            l.close()
    return out


def run_gpu_arm(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    from paged_infer_b200 import api
    from paged_infer_b200.loader import LlamaConfig

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    hbm_peak, peak_kind = measured_peaks()
    cfgd = dict(TINYLLAMA)
    cfg = LlamaConfig(**cfgd, quantization="int8")
    K, W = args.steps, max(args.warmup, 3)
    B = 64

    # A stream of our own (torch's default stream has handle 0, which the library reads as "create one").
    tstream = torch.cuda.Stream()
    torch.cuda.set_stream(tstream)
    ctx = api.Context(local_rank, stream=tstream.cuda_stream)
    model = api.LlamaWeights.synthetic(ctx, cfg, seed=0, std=0.02, max_batch=B, max_positions=4096)
    weight_bytes = model.weight_bytes()

    # --- resident run: K steps in one call -------------------------------------------------------------------
    pb = PagedBatch(2 + rank, B, 2 * (K + W) + 4)
    kv = api.KvCache(ctx, model.kv_layout(pb.num_blocks, BLOCK))
    kv.fill_normal(1234 + rank, 1.0)
    rng = np.random.default_rng(100 + rank)
    tokens = rng.integers(0, cfg.vocab_size, B).astype(np.uint32)

    def reserve(steps):  # pre-extend the tables so that `steps` device-side steps have writable slots
        saved = list(pb.lengths)
        for _ in range(steps):
            for src, dst in pb.plan():
                kv.copy_block(src, dst)
            pb.commit()
        pb.lengths = saved

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    reserve(W + K)
    out = model.decode_multi(tokens, pb.lengths, pb.tables, kv, W)       # warm-up steps
    tokens = out[-1].copy()
    pb.lengths = [n + W for n in pb.lengths]
    kv_tokens_unique = pb.unique_mapped_tokens()
    kv_tokens_logical = pb.logical_tokens()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    barrier()
    ctx.reset_kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    e0.record()
    out = model.decode_multi(tokens, pb.lengths, pb.tables, kv, K)
    e1.record()
    barrier()
    t_wall1 = time.time()
    launches = ctx.kernel_launches()
    resident_ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t_wall0, t_wall1)
    tokens = out[-1].copy()
    pb.lengths = [n + K for n in pb.lengths]

    # --- end to end: one public call per step, host bookkeeping + copies inside the timed region -----------------
    pb2 = PagedBatch(2 + rank, B, 2 * (K + W) + 4)
    pb2.pack(api)
    kv2 = kv  # same pool size and contents distribution; tables index the same physical range
    tok2 = rng.integers(0, cfg.vocab_size, B).astype(np.uint32)
    h2d = d2h = 0

    def e2e_step(tok):
        for src, dst in pb2.plan():
            kv2.copy_block(src, dst)
        ids = model.decode_batch_into(tok, pb2.lengths, pb2.packed, kv2, want_logits=False, want_argmax=True)
        pb2.commit()
        return ids

    for _ in range(W):
        tok2 = e2e_step(tok2)
    barrier()
    e0.record()
    for _ in range(K):
        tok2 = e2e_step(tok2)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    mb = max(len(t) for t in pb2.tables)
    h2d = B * mb * 4 + 3 * B * 4 + B * 4
    d2h = B * 4

    times = torch.tensor([resident_ms, e2e_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    resident_ms, e2e_ms = float(times[0]), float(times[1])

    # --- dominant kernel alone (rank 0) ----------------------------------------------------------------------------
    roof = other = gemv = cpu = profile_shares = None
    batch1 = prefill = None
    if rank == 0:
        H, hd, KH, NL = cfg.num_attention_heads, cfg.head_dim, cfg.num_key_value_heads, cfg.num_hidden_layers
        # Every launch of P real decode steps bracketed by CUDA events on the launching stream.
        P = min(K, 8)
        reserve(P)
        ctx.profile_begin()
        out = model.decode_multi(tokens, pb.lengths, pb.tables, kv, P)
        prof = ctx.profile_end()
        pb.lengths = [n + P for n in pb.lengths]
        total_ms = sum(ms for ms, _ in prof.values()) or 1e-9
        kv_bytes_layer = pb.unique_mapped_tokens() * KH * 2 * hd * 4
        algo = {"attention": kv_bytes_layer + 2 * B * H * hd * 4,
                "gemv": weight_bytes / max(prof["gemv"][1] / P, 1), "gemm_tc": weight_bytes / max(prof["gemm_tc"][1] / P, 1)}
        names = {"attention": "attn_decode_v3_kernel<64,8,3> (+ split merge): one layer, 64 sequences",
                 "gemv": "gemv_kernel<int8>: CUDA-core dequant projections of the step (average over the 5 matrices per layer)",
                 "gemm_tc": "gemm_ta_kernel<64,4> (+ the activation splits left): tcgen05 dequant projections of the step (average over its 89 launches)"}
        rl = {}
        for cls in ("attention", "gemv", "gemm_tc"):
            ms, n = prof[cls]
            if n == 0:
                continue
            us_serial = ms * 1e3 / n
            # inside the timed region launches overlap their predecessor's tail (programmatic dependent launch); the
            # events that bracket every launch here serialise them.  Duration inside the step = this class's share
            # of the bracketed device time x the step time of the timed region / its launches per step.
            us = (ms / total_ms) * (resident_ms / K) * 1e3 / (n / P)
            rl[cls] = {"kernel": names[cls], "bound": "hbm", "achieved": round(algo[cls] / us / 1e3, 1), "peak": hbm_peak,
                       "unit": "GB/s", "frac": round(algo[cls] / us / 1e3 / hbm_peak, 3),
                       "traffic": int(NCU_TRAFFIC_RATIO[cls] * algo[cls]),
                       "traffic_source": f"ncu dram bytes of a single-kernel capture scaled by algorithmic bytes (x{NCU_TRAFFIC_RATIO[cls]})",
                       "us_per_launch": round(us, 2), "us_per_launch_bracketed": round(us_serial, 2), "launches_per_step": n / P, "algorithmic_bytes_per_launch": int(algo[cls]),
                       "share_of_step_device_time": round(ms / total_ms, 3), "peak_kind": f"of {peak_kind}",
                       "timing": f"CUDA events around each of {n} launches inside {P} decode steps give the class's share; "
                                 "x the CUDA-event step time of the timed region / launches per step"}
        order = sorted(rl, key=lambda c: -rl[c]["share_of_step_device_time"])
        roof = rl[order[0]] if order else None
        other = [rl[c] for c in order[1:]]
        profile_shares = {c: round(ms / total_ms, 3) for c, (ms, _) in prof.items() if ms > 0}
        gemv = gemv_sweep(api, ctx, torch, hbm_peak)

        # batch-1 decode (config 0 shape): 128 greedy steps from position 128
        t1 = [list(range(0, 17))]
        kvb1 = api.KvCache(ctx, model.kv_layout(20, BLOCK))
        kvb1.fill_normal(5, 1.0)
        model.decode_multi([1], [128], t1, kvb1, 8)
        torch.cuda.synchronize()
        e0.record()
        model.decode_multi([1], [128], t1, kvb1, 128)
        e1.record()
        torch.cuda.synchronize()
        ms1 = e0.elapsed_time(e1) / 128
        bytes1 = weight_bytes + (128 + 64 + 1) * KH * 2 * hd * 4 * NL
        batch1 = {"tok/s": round(1e3 / ms1, 1), "ms_per_step": round(ms1, 4), "roofline_tok/s": round(hbm_peak * 1e9 / bytes1, 1),
                  "frac_of_hbm_roofline": round((bytes1 / (ms1 / 1e3)) / (hbm_peak * 1e9), 3), "bytes_per_step": bytes1}

        # prefill (config 0: 128-token prompt; config 4 style: 2048-token prompt), a model instance with room for
        # 512-position chunks; the chunk's attention runs in the shared-table kernel from 256 positions on
        prefill = {}
        pmodel = api.LlamaWeights.synthetic(ctx, cfg, seed=0, std=0.02, max_batch=512, max_positions=4096)
        for n_prompt, chunk in ((128, 128), (2048, 512)):
            nbp = n_prompt // BLOCK + 1
            kvp = api.KvCache(ctx, pmodel.kv_layout(nbp, BLOCK))
            prompt = np.random.default_rng(7).integers(0, cfg.vocab_size, n_prompt).astype(np.uint32)
            tab = list(range(nbp))
            pmodel.prefill_batched(prompt, 0, tab, kvp, chunk)
            torch.cuda.synchronize()
            reps = 3
            e0.record()
            for _ in range(reps):
                pmodel.prefill_batched(prompt, 0, tab, kvp, chunk)
            e1.record()
            torch.cuda.synchronize()
            msp = e0.elapsed_time(e1) / reps
            flops = 2.0 * n_prompt * (weight_bytes - cfg.vocab_size * cfg.hidden_size) + 4.0 * NL * H * hd * n_prompt * (n_prompt + 1) / 2
            prefill[f"prompt{n_prompt}_chunk{chunk}"] = {"tok/s": round(n_prompt / (msp / 1e3), 1), "ms": round(msp, 3),
                                                        "useful_TFLOP/s": round(flops / (msp / 1e3) / 1e12, 1)}
            kvp.close()
        pmodel.close()

        if world == 1 and not args.no_cpu:
            pbc = PagedBatch(2, B, 16)
            ts, threads, backend = cpu_decode_sample(cfgd, pbc, budget_s=20.0, max_steps=4)
            cms = float(np.mean(ts))
            cpu = {"value": round(B / cms, 2), "unit": "tok/s", "cores": threads, "kind": "port",
                   "sample": f"{len(ts)} full 64-sequence engine steps (same contexts and tables) on the CPU oracle, {backend}, {threads} threads"}

    if rank == 0:
        step_ms = resident_ms / K
        kv_bytes = kv_tokens_unique * cfg.num_key_value_heads * 2 * cfg.head_dim * 4 * cfg.num_hidden_layers
        step_bytes = weight_bytes + kv_bytes
        line = {
            "metric": "int8 batched paged decode throughput (TinyLlama-1.1B arch, 64 sequences)",
            "value": world * B * K / (resident_ms / 1e3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 weights, f32 activations/accumulate/KV", "data": "synthetic",
            "config": {"workload": "tinyllama_b64_paged", "batch_per_gpu": B, "block_size": BLOCK, "context": "U[256,2048] seed 2",
                       "prefix_shared_sequences": 32, "prefix_tokens": 512, "cow_forks": 8, "cow_copies": pb.total_cow + pb2.total_cow,
                       "lm_head": "int8", "weights": "N(0,0.02) generated on device, seed 0", "kv": "N(0,1) fill",
                       "parallelism": f"dp{world} (independent replicas, sequences sharded, no collective)" if world > 1 else "single GPU",
                       "l2": "inputs (1.04 GB weights + KV) are larger than L2; no flush needed"},
            "e2e": {"value": world * B * K / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / K},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": roof, "roofline_other": other, "device_time_shares": profile_shares,
            "step_roofline": {"bytes_per_step": step_bytes, "weight_bytes": weight_bytes, "kv_bytes_unique": kv_bytes,
                              "kv_tokens_unique": kv_tokens_unique, "kv_tokens_logical": kv_tokens_logical,
                              "achieved_GB/s": round(step_bytes / (step_ms / 1e3) / 1e9, 1), "peak_GB/s": hbm_peak,
                              "frac": round(step_bytes / (step_ms / 1e3) / 1e9 / hbm_peak, 3), "peak_kind": f"of {peak_kind}"},
            "gemv_m1": gemv, "batch1_decode": batch1, "prefill": prefill, "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


LLAMA3_8B = dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                 intermediate_size=14336, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)


LLAMA2_70B = dict(hidden_size=8192, num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
                  intermediate_size=28672, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)
TP_WORKLOADS = {
    # name: (architecture, model name, batch, contexts: fixed length or (lo, hi) uniform with the given seed)
    "llama3_8b_tp": (LLAMA3_8B, "Llama-3-8B", 32, 4096, 3),
    "llama2_70b_tp": (LLAMA2_70B, "Llama-2-70B", 64, (1024, 4096), 4),
}


def run_tp_workload(args, rank: int, world: int, local_rank: int):
    """`--workload llama3_8b_tp`: Llama-3-8B architecture, int8 projections, batch 32 decode at context 4096;
    `--workload llama2_70b_tp`: Llama-2-70B architecture, batch 64, contexts U[1024,4096] (needs >= 2 GPUs).
    Tensor-parallel over all `world` ranks (strong scaling: the total work is fixed)."""
    import torch
    import torch.distributed as dist

    from paged_infer_b200 import api
    from paged_infer_b200.loader import LlamaConfig
    from paged_infer_b200.tp import enable_peer_exchange, exchange_unique_id

    torch.cuda.set_device(local_rank)
    ident = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        ident = exchange_unique_id(api.nccl_unique_id, dist)
    hbm_peak, peak_kind = measured_peaks()
    arch, model_name, B, ctx_spec, seed = TP_WORKLOADS[args.workload]
    cfg = LlamaConfig(**arch, quantization="int8")
    K, W = args.steps, max(args.warmup, 3)
    rng = np.random.default_rng(seed)
    if isinstance(ctx_spec, tuple):
        ctx_len = [int(c) for c in rng.integers(ctx_spec[0], ctx_spec[1] + 1, B)]    # identical on every rank
        ctx_text = f"U[{ctx_spec[0]},{ctx_spec[1]}] seed {seed}"
    else:
        ctx_len = [ctx_spec] * B
        ctx_text = str(ctx_spec)
    CTX = max(ctx_len)
    tstream = torch.cuda.Stream()
    torch.cuda.set_stream(tstream)
    ctx = api.Context(local_rank, stream=tstream.cuda_stream, rank=rank, tp=world, nccl_id=ident)
    exchange = "single GPU"
    if world > 1:
        exchange = "nccl all-reduce"
        if not args.nccl_exchange:
            enable_peer_exchange(ctx, B * cfg.hidden_size, dist)
            exchange = "peer memory (P2P loads + flags, residual add folded in)"
    model = api.LlamaWeights.synthetic(ctx, cfg, seed=seed, std=0.02, max_batch=B, max_positions=CTX + K + W + 8)
    nblk = [(c + K + W + BLOCK) // BLOCK + 1 for c in ctx_len]
    first = np.concatenate([[0], np.cumsum(nblk)]).astype(int)
    kv = api.KvCache(ctx, model.kv_layout(int(first[-1]), BLOCK))
    kv.fill_normal(77 + rank, 1.0)
    tables = [list(range(int(first[b]), int(first[b + 1]))) for b in range(B)]
    tokens = rng.integers(0, cfg.vocab_size, B).astype(np.uint32)   # identical on every rank
    pos = list(ctx_len)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out = model.decode_multi(tokens, pos, tables, kv, W)
    tokens, pos = out[-1].copy(), [p + W for p in pos]
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    barrier()
    ctx.reset_kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    out = model.decode_multi(tokens, pos, tables, kv, K)
    e1.record()
    barrier()
    t1 = time.time()
    launches = ctx.kernel_launches()
    clocks = sampler.stop(t0, t1)
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms[0])
    # one profiled pass for the per-class shares (rank 0's view)
    ctx.profile_begin()
    model.decode_multi(out[-1].copy(), [p + K for p in pos], tables, kv, 2)
    prof = ctx.profile_end()
    if rank == 0:
        total = sum(v[0] for v in prof.values()) or 1e-9
        weight_bytes = model.weight_bytes()                         # this rank's shard
        kv_bytes = sum(c + W + K // 2 for c in ctx_len) * (cfg.num_key_value_heads // world) * 2 * cfg.head_dim * 4 * cfg.num_hidden_layers
        step_ms = ms / K
        line = {
            "metric": f"int8 batched paged decode throughput ({model_name} arch, batch {B}, context {ctx_text}, tensor parallel)",
            "value": B * K / (ms / 1e3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 weights, f32 activations/accumulate/KV", "data": "synthetic",
            "config": {"workload": args.workload, "batch": B, "context": ctx_text, "block_size": BLOCK, "parallelism": f"tp{world}",
                       "collectives_per_step": 2 * cfg.num_hidden_layers + 1 if world > 1 else 0, "exchange": exchange,
                       "weights": f"N(0,0.02) generated on device, seed {seed}", "kv": "N(0,1) fill"},
            "gpu_launches": launches, "clocks": clocks,
            "step_roofline": {"bytes_per_step_per_gpu": weight_bytes + kv_bytes, "weight_bytes_per_gpu": weight_bytes,
                              "kv_bytes_per_gpu": kv_bytes, "achieved_GB/s_per_gpu": round((weight_bytes + kv_bytes) / (step_ms / 1e3) / 1e9, 1),
                              "peak_GB/s": hbm_peak, "frac": round((weight_bytes + kv_bytes) / (step_ms / 1e3) / 1e9 / hbm_peak, 3),
                              "peak_kind": f"of {peak_kind}"},
            "device_time_shares": {c: round(v[0] / total, 3) for c, v in prof.items() if v[0] > 0},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_kernel_case(args):
    """`--kernel-case NAME`: a handful of launches of ONE kernel on a small case of the default workload's shapes,
    for a profiler to capture (the numbers it prints itself are CUDA-event times of the same launches)."""
    import torch

    from paged_infer_b200 import api
    from paged_infer_b200.loader import LlamaConfig

    torch.cuda.set_device(0)
    tstream = torch.cuda.Stream()
    torch.cuda.set_stream(tstream)
    ctx = api.Context(0, stream=tstream.cuda_stream)
    rng = np.random.default_rng(11)
    reps = max(args.steps, 1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    case = args.kernel_case
    if case in ("gemv_lm_head", "gemm_lm_head", "gemm_gate_up", "gemm_down"):
        M = 1 if case.startswith("gemv") else 64
        N, Kc = {"gemv_lm_head": (32000, 2048), "gemm_lm_head": (32000, 2048), "gemm_gate_up": (11264, 2048),
                 "gemm_down": (2048, 5632)}[case]
        q = rng.integers(-127, 128, (N, Kc), dtype=np.int8)
        s = np.full(N, 1.6e-4, np.float32)
        copies = 4                                            # rotate so that no launch finds its weights in L2
        lins = [api.Projection.int8(ctx, q, s) for _ in range(copies)]
        x = torch.randn(M, Kc, device="cuda", dtype=torch.float32)
        y = torch.empty(M, N, device="cuda", dtype=torch.float32)
        for l in lins:
            l.apply_device(x, y, M)
        torch.cuda.synchronize()
        e0.record()
        for r in range(reps):
            lins[r % copies].apply_device(x, y, M)
        e1.record()
        torch.cuda.synchronize()
        algo = N * Kc + 4 * N + 4 * M * Kc + 4 * M * N
    elif case == "attention":
        cfg = LlamaConfig(**TINYLLAMA, quantization="int8")
        B, ctx_len = 64, 1024
        nblk = ctx_len // BLOCK + 1
        layout = api.KvLayout(1, B * nblk, BLOCK, cfg.num_key_value_heads, cfg.head_dim)
        kv = api.KvCache(ctx, layout)
        kv.fill_normal(9, 1.0)
        attn = api.PagedAttention(layout, cfg.num_attention_heads)
        qv = torch.randn(B, cfg.num_attention_heads * cfg.head_dim, device="cuda", dtype=torch.float32)
        ov = torch.empty_like(qv)
        entries = [api.AttnEntry(api.BlockTable(list(range(b * nblk, (b + 1) * nblk))), ctx_len - 1) for b in range(B)]
        attn.run_device(qv, ov, kv, entries)
        torch.cuda.synchronize()
        e0.record()
        for r in range(reps):
            attn.run_device(qv, ov, kv, entries)
        e1.record()
        torch.cuda.synchronize()
        algo = B * ctx_len * cfg.num_key_value_heads * 2 * cfg.head_dim * 4 + 2 * qv.numel() * 4
    elif case == "attention_prefill":
        # the last 512-position chunk of a 2048-token prompt: every entry maps the same table
        cfg = LlamaConfig(**TINYLLAMA, quantization="int8")
        n_ctx, chunk = 2048, 512
        nblk = n_ctx // BLOCK
        layout = api.KvLayout(1, nblk, BLOCK, cfg.num_key_value_heads, cfg.head_dim)
        kv = api.KvCache(ctx, layout)
        kv.fill_normal(9, 1.0)
        attn = api.PagedAttention(layout, cfg.num_attention_heads)
        qv = torch.randn(chunk, cfg.num_attention_heads * cfg.head_dim, device="cuda", dtype=torch.float32)
        ov = torch.empty_like(qv)
        table = api.BlockTable(list(range(nblk)))
        entries = [api.AttnEntry(table, n_ctx - chunk + i) for i in range(chunk)]
        attn.run_device(qv, ov, kv, entries)
        torch.cuda.synchronize()
        ctx.profile_begin()                      # device time of the launches only: packing 512 tables on the host is slow
        for r in range(reps):
            attn.run_device(qv, ov, kv, entries)
        prof = ctx.profile_end()
        us = prof["attention"][0] * 1e3 / max(prof["attention"][1], 1)
        pairs = sum(n_ctx - chunk + i + 1 for i in range(chunk))          # (position, token) pairs inside the windows
        flops = 4.0 * pairs * cfg.num_attention_heads * cfg.head_dim
        print(json.dumps({"kernel_case": case, "launches": prof["attention"][1], "us_per_launch": round(us, 2), "useful_flops": flops,
                          "useful_TFLOP/s": round(flops / us / 1e6, 2),
                          "note": "every f32 product is carried by six bf16 x bf16 tensor-core products (three planes per operand)"}),
              flush=True)
        return
    else:
        raise SystemExit(f"unknown kernel case {case}")
    us = e0.elapsed_time(e1) * 1e3 / reps
    hbm_peak, peak_kind = measured_peaks()
    print(json.dumps({"kernel_case": case, "launch_groups": reps, "us_per_launch_group": round(us, 2),
                      "algorithmic_bytes": int(algo), "GB/s": round(algo / us / 1e3, 1),
                      "frac_of_hbm_peak": round(algo / us / 1e3 / hbm_peak, 3), "peak_kind": f"of {peak_kind}"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel-case", default=None,
                    choices=["gemv_lm_head", "gemm_lm_head", "gemm_gate_up", "gemm_down", "attention", "attention_prefill"],
                    help="run a few launches of one kernel on a small case (for a profiler) and exit")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="tinyllama_b64_paged", choices=["tinyllama_b64_paged", "llama3_8b_tp", "llama2_70b_tp"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--nccl-exchange", action="store_true", help="llama3_8b_tp: all-reduce through NCCL instead of the peer-memory kernel")
    args = ap.parse_args()
    # stdout carries exactly one JSON line: NCCL's own banner ("NCCL version ...") goes to stderr
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.kernel_case:
        run_kernel_case(args)
        return
    if args.workload in TP_WORKLOADS:
        run_tp_workload(args, rank, world, local_rank)
        return
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
