#!/usr/bin/env python3
"""Benchmark of the int8 paged-decode hot path on B200.

Default workload (`tinyllama_b64_paged`): TinyLlama-1.1B architecture, random-init
int8 projections (lm_head int8 as well), 64 concurrent sequences with context
lengths uniform in [256, 2048] (seed 2), KV block size 16, f32 KV.  The batch is
set up the way the engine would: every prompt is admitted through the C++
KvCacheManager (chained block hash: sequences 0-31 share the first 512 token
ids and therefore the same 32 physical blocks), prefilled on the device for the
part the prefix cache did not cover, published; sequences 56-63 are forks of
48-55 (same table, copy-on-write split on their first write).  A "step" is one
engine step: one greedy decode token for each of the 64 sequences.

  value      decode tok/s with everything resident on the device: K greedy steps
             inside one `pi_model_decode_multi` call (no host round trip between
             steps), timed with CUDA events.
  e2e        the same metric through the per-step public call
             (`LlamaWeights.decode_batch_into`): block bookkeeping by the
             KvCacheManager on the host (grow, copy-on-write), tokens / tables /
             positions copied host->device and the chosen ids device->host
             inside the timed region, every step.
  roofline   the dominant kernel class timed with CUDA events inside real steps.
  cpu_baseline  the CPU oracle (a C++ restatement of the reference's rayon/AVX2
             path; the reference itself is Rust and cannot be built here) on a
             bounded sample of the same workload, on this box's host cores.

`--impl reference` times that CPU path as the reference arm.  With `--gpus N`
under torchrun every rank first runs its own replica of the workload (sequences
are independent; no collective on the data path: weak scaling, `value`), then
all N ranks together run the tensor-parallel workload of the sharded
configuration (Llama-3-8B architecture, batch 32, context 4096: column-split
q/k/v/gate/up, row-split o/down with one exchange each) and attach it as `tp`.
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


# ---- the batch as the engine holds it ---------------------------------------------------------------------------
class EngineBatch:
    """The 64 sequences of the workload with their block bookkeeping done by the C++ KvCacheManager
    (include/paged_infer_memory.hpp behind libpaged_infer_host.so; reference src/memory/kv_cache_manager.rs:116-345):
    admission with prefix reuse through the chained block hash, publishing, forks, and before every step
    ``prepare_step`` = Engine::plan_step (src/engine.rs:612-699): grow the mapping, split shared blocks copy-on-write.
    The tables live in the packed arrays that the device library takes and are updated in place."""

    def __init__(self, api, seed: int, batch: int, reserve_steps: int, lo=256, hi=2048, prefix_tokens=512, forks=8, vocab=32000):
        from paged_infer_b200 import host
        rng = np.random.default_rng(seed)
        ctx = rng.integers(lo, hi + 1, batch)
        if forks:
            ctx[batch - forks:] = ctx[batch - 2 * forks:batch - forks]   # a fork starts at its parent's length
        self.batch, self.forks, self.prefix_tokens = batch, forks, prefix_tokens
        self.lengths = np.array(ctx, np.int32)
        prefix = rng.integers(0, vocab, prefix_tokens).astype(np.uint32)
        self.prompts = []
        for b in range(batch - forks):
            n = int(ctx[b])
            if b < batch // 2:   # the first half of the batch opens with the same token ids
                t = np.concatenate([prefix, rng.integers(0, vocab, max(n - prefix_tokens, 0)).astype(np.uint32)])[:n]
            else:
                t = rng.integers(0, vocab, n).astype(np.uint32)
            self.prompts.append(t)
        self.num_blocks = int(sum((int(c) + reserve_steps) // BLOCK + 2 for c in ctx)) + 64
        self.mgr = host.KvCacheManager(self.num_blocks, BLOCK, True)
        width = (int(ctx.max()) + reserve_steps) // BLOCK + 4
        self.packed = api.PackedBlockTables(batch, width) if api is not None else None
        self.tables = self.packed.mat if api is not None else np.full((batch, width), -1, np.int32)
        self.lens = self.packed.lens if api is not None else np.zeros(batch, np.int32)
        self.cow = np.empty((batch, 2), np.int32)
        self.seq_ids = np.arange(batch, dtype=np.uint64)
        self.tick = 0
        self.prefilled_tokens = 0

    def admit_all(self, prefill=None):
        """Admit, prefill what the prefix cache did not cover (``prefill(tokens, start_pos, table)``; None: bookkeeping
        only) and publish every prompt, in order; then fork the last sequences from their parents."""
        for b in range(self.batch - self.forks):
            prompt = self.prompts[b]
            cached = self.mgr.admit(b, prompt, self.tick)
            resume = min(cached, len(prompt) - 1)    # a fully cached prompt still recomputes its last token
            if prefill is not None:
                prefill(prompt[resume:], resume, self.mgr.table(b))
            self.prefilled_tokens += len(prompt) - resume
            self.mgr.publish_prompt_blocks(b)
        for i in range(self.forks):
            self.mgr.fork(self.batch - 2 * self.forks + i, self.batch - self.forks + i, self.tick)

    def plan(self, ahead: int = 0):
        """Settle memory for the step that writes position length + ahead of every sequence; -> [(src, dst)] copies."""
        self.tick += 1
        pos = (self.lengths + ahead).astype(np.int32)
        n = self.mgr.prepare_step(self.seq_ids, pos, self.tables, self.lens, self.cow, self.tick)
        return [(int(self.cow[i, 0]), int(self.cow[i, 1])) for i in range(n)]

    def commit(self, steps: int = 1):
        self.lengths += steps

    def table_lists(self):
        return [self.tables[b, :self.lens[b]].tolist() for b in range(self.batch)]

    def unique_mapped_tokens(self) -> int:
        """Tokens of KV that one step must read at least once (shared physical blocks count once)."""
        seen = {}
        for b in range(self.batch):
            n = int(self.lengths[b])
            for lb in range(int(self.lens[b])):
                used = min(BLOCK, n + 1 - lb * BLOCK)
                if used > 0:
                    pb = int(self.tables[b, lb])
                    seen[pb] = max(seen.get(pb, 0), used)
        return sum(seen.values())

    def logical_tokens(self) -> int:
        return int((self.lengths + 1).sum())


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


def measured_peaks(sustained: bool = False):
    """(HBM GB/s, dense bf16 TFLOP/s, kind): the driver-measured peaks of this pool, else the stated fallback.  The bf16
    figure is the burst one for a kernel timed alone, the sustained one for a kernel timed inside a long step."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained" if sustained else "bf16_tflops"]), "measured"
    return 6650.0, (1400.0 if sustained else 1590.0), "fallback"


# ---- the CPU arm (oracle) ---------------------------------------------------------------------------------------
def cpu_decode_sample(cfg: dict, eb: EngineBatch, budget_s: float, max_steps: int, warmup: int = 1):
    """Time oracle decode steps of the same 64 sequences (same tables, from the same KvCacheManager) on the host cores.
    The thread count is set here to the cores this process may run on, whatever the launcher put in OMP_NUM_THREADS."""
    from oracle import pi_oracle as orc
    orc.build()
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    orc.lib().orc_set_num_threads(int(cores))
    rng = np.random.default_rng(7)
    H, NL, KH = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_key_value_heads"]
    hd = H // cfg["num_attention_heads"]
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]

    def i8(rows, cols):
        return (rng.integers(-127, 128, (rows, cols), dtype=np.int8), np.full(rows, 1.6e-4, np.float32))

    shapes = {"wq": (H, H), "wk": (KH * hd, H), "wv": (KH * hd, H), "wo": (H, H), "w1": (inter, H), "w2": (H, inter), "w3": (inter, H)}
    projs = [{k: i8(*s) for k, s in shapes.items()} for _ in range(NL)]   # every layer its own codes: 1 GB streamed per step
    embed = rng.integers(0x3B00, 0x3C00, (vocab, H), dtype=np.uint16)  # small positive bf16 values
    ones = np.ones(H, np.float32)
    model = orc.Model(cfg, embed, ones, [ones] * NL, [ones] * NL, projs, i8(vocab, H))
    layout_floats = NL * eb.num_blocks * BLOCK * KH * 2 * hd
    chunk = rng.standard_normal(1 << 22).astype(np.float32)
    kv = np.resize(chunk, layout_floats)     # values do not change the CPU path's timing; the tables are the real ones
    olayout = orc.kv_layout(NL, eb.num_blocks, BLOCK, KH, hd)
    tokens = rng.integers(0, vocab, eb.batch).astype(np.uint32)
    times = []
    t_start = time.time()
    for s in range(warmup + max_steps):
        t0 = time.perf_counter()
        for src, dst in eb.plan():
            orc.kv_copy_block(olayout, kv, src, dst)
        logits = model.decode_batch(tokens, eb.lengths.tolist(), eb.table_lists(), kv, BLOCK)
        tokens = np.array([orc.argmax(r) for r in logits], np.uint32)
        dt = time.perf_counter() - t0
        eb.commit()
        if s >= warmup:
            times.append(dt)
        if time.time() - t_start > budget_s and len(times) >= 1:
            break
    return times, orc.num_threads(), orc.backend()


def workload_config(eb: EngineBatch, extra: dict) -> dict:
    """The `config` object both arms print: same keys, same workload."""
    st = eb.mgr.stats()
    cfg = {"workload": "tinyllama_b64_paged", "batch_per_gpu": eb.batch, "block_size": BLOCK, "context": "U[256,2048] seed 2",
           "prefix_shared_sequences": eb.batch // 2, "prefix_tokens": eb.prefix_tokens, "cow_forks": eb.forks,
           "host_bookkeeping": "C++ KvCacheManager (admit -> prefill tail -> publish -> fork -> prepare_step)",
           "prefix_cache_hits": st["prefix_hits"], "prefix_tokens_saved": st["prefix_tokens_saved"], "cow_copies": st["cow_copies"],
           "lm_head": "int8"}
    cfg.update(extra)
    return cfg


def run_reference_arm(args, rank: int):
    if rank != 0:
        return
    cfg = dict(TINYLLAMA)
    W = max(args.warmup, 1)
    eb = EngineBatch(None, 2, 64, args.steps + W + 4)
    eb.admit_all(None)
    times, threads, backend = cpu_decode_sample(cfg, eb, budget_s=150.0, max_steps=args.steps, warmup=W)
    ms = 1e3 * float(np.mean(times))
    val = 64.0 / (ms / 1e3)
    sample = (f"{len(times)} of the requested {args.steps} steps (time-bounded, {W} warm-up), each a full 64-sequence engine step "
              f"(contexts U[256,2048], block 16, 22 distinct layers of int8 codes) on the CPU oracle, {backend}, {threads} threads")
    line = {
        "impl": "reference", "metric": "int8 batched paged decode throughput (TinyLlama-1.1B arch, 64 sequences)",
        "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": len(times), "warmup": W,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 weights, f32 activations/accumulate/KV",
        "data": "synthetic",
        "config": workload_config(eb, {"weights": "uniform int8 codes, 22 distinct layers", "kv": "N(0,1) fill (timing does not depend on the values)",
                                       "parallelism": "host cores"}),
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


def config1_sweep(api, ctx, torch, hbm_peak, bf16_peak, reps=3):
    """The isolated projection sweep of the second configuration: every TinyLlama projection shape at 1, 8, 32, 128
    and 512 activation rows.  Weight copies rotate so that every launch streams its weights from HBM; launches go
    back to back with one CUDA-event pair around the train.  Up to 32 rows the figure is GB/s over the algorithmic
    bytes (HBM bound); from 128 rows on it is useful TFLOP/s (2*M*N*K) against the measured bf16 peak - the tensor
    pipe does three times that work because every f32 activation travels as three bf16 planes."""
    out = {}
    rng = np.random.default_rng(1)
    shapes = {k: v for k, v in GEMV_SHAPES.items() if "Llama-3" not in k and "fused" not in k}
    for name, (N, K) in shapes.items():
        bytes_w = N * K + 4 * N
        copies = int(min(24, max(2, -(-(300 << 20) // bytes_w))))
        q = rng.integers(-127, 128, (N, K), dtype=np.int8)
        sc = np.full(N, 1.6e-4, np.float32)
        lins = [api.Projection.int8(ctx, q, sc) for _ in range(copies)]
        row = {}
        for M in (1, 8, 32, 128, 512):
            x = torch.randn(M, K, device="cuda", dtype=torch.float32)
            y = torch.empty(M, N, device="cuda", dtype=torch.float32)
            for l in lins:
                l.apply_device(x, y, M)
            torch.cuda.synchronize()
            best = None
            rounds = 2 if M >= 128 else 4
            for _ in range(reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _r in range(rounds):
                    for l in lins:
                        l.apply_device(x, y, M)
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (rounds * copies)
                best = us if best is None else min(best, us)
            algo = N * K + 4 * N + 4 * M * K + 4 * M * N
            ent = {"us": round(best, 2), "GB/s": round(algo / best / 1e3, 1), "frac_of_hbm_peak": round(algo / best / 1e3 / hbm_peak, 3)}
            if M >= 128:
                tf = 2.0 * M * N * K / best / 1e6
                ent.update({"useful_TFLOP/s": round(tf, 1), "frac_of_bf16_peak": round(tf / bf16_peak, 3),
                            "tensor_TFLOP/s_with_3_planes": round(3 * tf, 1)})
            row[f"M={M}"] = ent
        out[name] = row
        for l in lins:
            l.close()
    return out


def prefill_70b_shape(api, ctx, torch, layers=2):
    """The prefill batch of the 70B configuration - 8 prompts of 2048 tokens at hidden 8192, 64 query / 8 KV heads of
    128, FFN 28672 - on a model cut to `layers` layers (one GPU holds them; the full model is 80 of the same), chunks
    of 512 positions.  Device-generated int8 weights."""
    from paged_infer_b200.loader import LlamaConfig
    arch = dict(LLAMA2_70B)
    arch["num_hidden_layers"] = layers
    cfg = LlamaConfig(**arch, quantization="int8")
    model = api.LlamaWeights.synthetic(ctx, cfg, seed=4, std=0.02, max_batch=512, max_positions=2048 + 16)
    n_prompt, prompts, chunk = 2048, 8, 512
    nbp = n_prompt // BLOCK + 1
    kv = api.KvCache(ctx, model.kv_layout(prompts * nbp, BLOCK))
    rng = np.random.default_rng(4)
    toks = [rng.integers(0, cfg.vocab_size, n_prompt).astype(np.uint32) for _ in range(prompts)]
    tabs = [list(range(i * nbp, (i + 1) * nbp)) for i in range(prompts)]
    model.prefill_batched(toks[0], 0, tabs[0], kv, chunk)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for t, tab in zip(toks, tabs):
        model.prefill_batched(t, 0, tab, kv, chunk)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    layer_weights = model.weight_bytes() - cfg.vocab_size * cfg.hidden_size - 4 * cfg.vocab_size
    H, hd = cfg.num_attention_heads, cfg.head_dim
    flops = prompts * (2.0 * n_prompt * layer_weights + 4.0 * layers * H * hd * n_prompt * (n_prompt + 1) / 2)
    out = {"layers": layers, "of_layers": 80, "prompts": prompts, "prompt_tokens": n_prompt, "chunk": chunk, "ms": round(ms, 2),
           "tok/s_at_this_depth": round(prompts * n_prompt / (ms / 1e3), 1), "ms_per_layer_per_prompt": round(ms / layers / prompts, 3),
           "useful_TFLOP/s": round(flops / (ms / 1e3) / 1e12, 1),
           "attention": "head_dim 128: shared-table kernel on mma.sync TF32x3 (the tcgen05 one covers head_dim 64)"}
    kv.close()
    model.close()
    return out


def run_gpu_arm(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    from paged_infer_b200 import api
    from paged_infer_b200.loader import LlamaConfig

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    cfgd = dict(TINYLLAMA)
    cfg = LlamaConfig(**cfgd, quantization="int8")
    K, W = args.steps, max(args.warmup, 3)
    B = 64
    P = min(K, 8)

    # A stream of our own (torch's default stream has handle 0, which the library reads as "create one").
    tstream = torch.cuda.Stream()
    torch.cuda.set_stream(tstream)
    ctx = api.Context(local_rank, stream=tstream.cuda_stream)
    if args.attn_grid:
        ctx.set_option(api._lib.PI_OPT_ATTN_FLAT, 0)
    model = api.LlamaWeights.synthetic(ctx, cfg, seed=0, std=0.02, max_batch=512, max_positions=4096)
    weight_bytes = model.weight_bytes()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # --- the batch, set up as the engine would: the same on every rank (same seed: replicas of one workload) ---------
    eb = EngineBatch(api, 2, B, 2 * (K + W) + P + 8, vocab=cfg.vocab_size)
    kv = api.KvCache(ctx, model.kv_layout(eb.num_blocks, BLOCK))
    t0 = time.time()
    if args.resident_only:     # profiler runs: bookkeeping only, N(0,1) values in the pool
        eb.admit_all(None)
        kv.fill_normal(1234, 1.0)
    else:
        eb.admit_all(lambda toks, start, table: model.prefill_batched(toks, start, table, kv, 512))
    torch.cuda.synchronize()
    setup_prefill_s = time.time() - t0
    rng = np.random.default_rng(100)
    tokens = rng.integers(0, cfg.vocab_size, B).astype(np.uint32)

    # --- end to end: one public call per step, host bookkeeping + copies inside the timed region --------------------
    def e2e_step(tok):
        for src, dst in eb.plan():
            kv.copy_block(src, dst)
        ids = model.decode_batch_into(tok, eb.lengths, eb.packed, kv, want_logits=False, want_argmax=True)
        eb.commit()
        return ids

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_ms = float("nan")
    if not args.resident_only:
        for _ in range(W):
            tokens = e2e_step(tokens)
        barrier()
        e0.record()
        for _ in range(K):
            tokens = e2e_step(tokens)
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)
    mb = int(eb.lens.max())
    h2d = B * mb * 4 + 3 * B * 4 + B * 4
    d2h = B * 4

    # --- resident run: K steps in one call ----------------------------------------------------------------------------
    def reserve(steps):  # pre-extend the tables so that `steps` device-side steps have writable slots
        for s in range(steps):
            for src, dst in eb.plan(ahead=s):
                kv.copy_block(src, dst)

    reserve(W + K)
    out = model.decode_multi(tokens, eb.lengths, eb.packed, kv, W)       # warm-up steps
    tokens = out[-1].copy()
    eb.commit(W)
    kv_tokens_unique = eb.unique_mapped_tokens()
    kv_tokens_logical = eb.logical_tokens()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    barrier()
    ctx.reset_kernel_launches()
    t_wall0 = time.time()
    e0.record()
    out = model.decode_multi(tokens, eb.lengths, eb.packed, kv, K)
    e1.record()
    barrier()
    t_wall1 = time.time()
    launches = ctx.kernel_launches()
    resident_ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t_wall0, t_wall1)
    tokens = out[-1].copy()
    eb.commit(K)

    mine = torch.tensor([resident_ms, e2e_ms], device="cuda", dtype=torch.float64)
    per_rank = [mine.clone() for _ in range(world)]
    if world > 1:
        dist.all_gather(per_rank, mine)
    resident_all = [float(t[0]) for t in per_rank]
    e2e_all = [float(t[1]) for t in per_rank]
    resident_ms, e2e_ms = max(resident_all), max(e2e_all)

    # --- kernel classes inside real steps, and the other configurations (rank 0) ------------------------------------
    roof = other = sweep = gemv = cpu = profile_shares = None
    batch1 = prefill = prefill70 = None
    if args.resident_only:
        if rank == 0:
            print(json.dumps({"resident_only": True, "ms_per_step": resident_ms / K, "gpu_launches": launches, "steps": K, "warmup": W}), flush=True)
        kv.close()
        model.close()
        ctx.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if rank == 0:
        H, hd, KH, NL = cfg.num_attention_heads, cfg.head_dim, cfg.num_key_value_heads, cfg.num_hidden_layers
        # Every launch of P real decode steps bracketed by CUDA events on the launching stream.
        reserve(P)
        ctx.profile_begin()
        out = model.decode_multi(tokens, eb.lengths, eb.packed, kv, P)
        prof = ctx.profile_end()
        eb.commit(P)
        total_ms = sum(ms for ms, _ in prof.values()) or 1e-9
        kv_bytes_layer = eb.unique_mapped_tokens() * KH * 2 * hd * 4
        algo = {"attention": kv_bytes_layer + 2 * B * H * hd * 4,
                "gemv": weight_bytes / max(prof["gemv"][1] / P, 1), "gemm_tc": weight_bytes / max(prof["gemm_tc"][1] / P, 1)}
        names = {"attention": "attn_decode_flat_kernel<64,8,3> (one layer, 64 sequences; the step's one attn_plan_kernel launch is spread over the layers)"
                              if not args.attn_grid else "attn_decode_v3_kernel<64,8,3> + attn_combine_kernel: one layer, 64 sequences",
                 "gemv": "gemv_kernel<int8>: CUDA-core dequant projections of the step",
                 "gemm_tc": "gemm_ta_kernel<64,4>: tcgen05 dequant projections of the step (average over its launches)"}
        rl = {}
        for cls in ("attention", "gemv", "gemm_tc"):
            ms, n = prof[cls]
            if n == 0:
                continue
            if cls == "attention":
                n = NL * P          # per layer: the work-list kernel (once per step) and the merge kernel are part of the layer's attention
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
            if cls == "gemm_tc":   # the same launches against the tensor roof: three bf16 planes per f32 activation
                rows_total = NL * (3 * cfg.hidden_size + 2 * KH * hd + 2 * cfg.intermediate_size) + cfg.vocab_size
                tf = 3 * 2.0 * B * (weight_bytes - 4 * rows_total) / (n / P) / us / 1e6
                rl[cls]["tensor_TFLOP/s_with_3_planes"] = round(tf, 1)
                rl[cls]["frac_of_bf16_sustained_peak"] = round(tf / measured_peaks(sustained=True)[1], 3)
        order = sorted(rl, key=lambda c: -rl[c]["share_of_step_device_time"])
        roof = rl[order[0]] if order else None
        other = [rl[c] for c in order[1:]]
        profile_shares = {c: round(ms / total_ms, 3) for c, (ms, _) in prof.items() if ms > 0}
        kv.close()

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
        # the same steps with CUDA events around every launch: what a projection costs INSIDE the step (the back-to-back
        # figures of `gemv_m1` have no dependent kernel ahead of them)
        ctx.profile_begin()
        model.decode_multi([1], [192], t1, kvb1, 16)
        prof1 = ctx.profile_end()
        tot1 = sum(ms for ms, _ in prof1.values()) or 1e-9
        batch1["in_step"] = {c: {"launches_per_step": n / 16, "share": round(ms / tot1, 3),
                                 "us_per_launch": round((ms / tot1) * ms1 * 1e3 / (n / 16), 2),
                                 "us_per_launch_bracketed": round(ms * 1e3 / n, 2)}
                             for c, (ms, n) in prof1.items() if n > 0}
        kvb1.close()

        # prefill (config 0: 128-token prompt; a 2048-token prompt in 512-position chunks)
        prefill = {"batch_setup": {"tokens_prefilled": eb.prefilled_tokens, "s": round(setup_prefill_s, 2),
                                   "note": "the 56 prompts of the default workload, prefix hits skipped, chunk 512, host loop included"}}
        for n_prompt, chunk in ((128, 128), (2048, 512)):
            nbp = n_prompt // BLOCK + 1
            kvp = api.KvCache(ctx, model.kv_layout(nbp, BLOCK))
            prompt = np.random.default_rng(7).integers(0, cfg.vocab_size, n_prompt).astype(np.uint32)
            tab = list(range(nbp))
            model.prefill_batched(prompt, 0, tab, kvp, chunk)
            torch.cuda.synchronize()
            reps = 3
            e0.record()
            for _ in range(reps):
                model.prefill_batched(prompt, 0, tab, kvp, chunk)
            e1.record()
            torch.cuda.synchronize()
            msp = e0.elapsed_time(e1) / reps
            flops = 2.0 * n_prompt * (weight_bytes - cfg.vocab_size * cfg.hidden_size) + 4.0 * NL * H * hd * n_prompt * (n_prompt + 1) / 2
            prefill[f"prompt{n_prompt}_chunk{chunk}"] = {"tok/s": round(n_prompt / (msp / 1e3), 1), "ms": round(msp, 3),
                                                        "useful_TFLOP/s": round(flops / (msp / 1e3) / 1e12, 1)}
            kvp.close()
        model.close()
        sweep = config1_sweep(api, ctx, torch, hbm_peak, bf16_peak)
        gemv = gemv_sweep(api, ctx, torch, hbm_peak)
        prefill70 = prefill_70b_shape(api, ctx, torch)

        if world == 1 and not args.no_cpu:
            ebc = EngineBatch(None, 2, B, 16)
            ebc.admit_all(None)
            ts, threads, backend = cpu_decode_sample(cfgd, ebc, budget_s=20.0, max_steps=4)
            cms = float(np.mean(ts))
            cpu = {"value": round(B / cms, 2), "unit": "tok/s", "cores": threads, "kind": "port",
                   "sample": f"{len(ts)} full 64-sequence engine steps (same contexts and tables) on the CPU oracle, {backend}, {threads} threads"}
    else:
        kv.close()
        model.close()
    ctx.close()

    # --- the sharded configuration over the same ranks -----------------------------------------------------------------
    tp = None
    if world > 1:
        barrier()
        tp = tp_decode(args, "llama3_8b_tp", rank, world, local_rank, min(K, 16), W, with_tp1=True)

    if rank == 0:
        step_ms = resident_ms / K
        kv_bytes = kv_tokens_unique * cfg.num_key_value_heads * 2 * cfg.head_dim * 4 * cfg.num_hidden_layers
        step_bytes = weight_bytes + kv_bytes
        line = {
            "metric": "int8 batched paged decode throughput (TinyLlama-1.1B arch, 64 sequences)",
            "value": world * B * K / (resident_ms / 1e3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 weights, f32 activations/accumulate/KV", "data": "synthetic",
            "config": workload_config(eb, {"weights": "N(0,0.02) generated on device, seed 0",
                                           "kv": "written by prefill of the 56 prompts (random token ids, seed 2)",
                                           "parallelism": f"dp{world} (independent replicas of the same batch, no collective)" if world > 1 else "single GPU",
                                           "l2": "inputs (1.04 GB weights + KV) are larger than L2; no flush needed"}),
            "e2e": {"value": world * B * K / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / K},
            "per_rank_ms_per_step": {"resident": [round(t / K, 4) for t in resident_all], "e2e": [round(t / K, 4) for t in e2e_all]},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": roof, "roofline_other": other, "device_time_shares": profile_shares,
            "step_roofline": {"bytes_per_step": step_bytes, "weight_bytes": weight_bytes, "kv_bytes_unique": kv_bytes,
                              "kv_tokens_unique": kv_tokens_unique, "kv_tokens_logical": kv_tokens_logical,
                              "achieved_GB/s": round(step_bytes / (step_ms / 1e3) / 1e9, 1), "peak_GB/s": hbm_peak,
                              "frac": round(step_bytes / (step_ms / 1e3) / 1e9 / hbm_peak, 3), "peak_kind": f"of {peak_kind}"},
            "config1_sweep": sweep, "gemv_m1": gemv, "batch1_decode": batch1, "prefill": prefill, "prefill_70b_shape": prefill70, "cpu_baseline": cpu,
            "tp": tp,
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


def tp_decode(args, workload: str, rank: int, world: int, local_rank: int, K: int, W: int, with_tp1: bool = False):
    """One tensor-parallel decode measurement over the `world` ranks of an initialised process group (strong scaling:
    the total work is fixed).  Returns the result on rank 0, None elsewhere.  `with_tp1`: rank 0 also runs the same
    workload alone on its GPU, for the speed-up."""
    import torch
    import torch.distributed as dist

    from paged_infer_b200 import api
    from paged_infer_b200.loader import LlamaConfig
    from paged_infer_b200.tp import enable_peer_exchange, exchange_unique_id

    hbm_peak, _, peak_kind = measured_peaks()
    arch, model_name, B, ctx_spec, seed = TP_WORKLOADS[workload]
    cfg = LlamaConfig(**arch, quantization="int8")
    rng = np.random.default_rng(seed)
    if isinstance(ctx_spec, tuple):
        ctx_len = [int(c) for c in rng.integers(ctx_spec[0], ctx_spec[1] + 1, B)]    # identical on every rank
        ctx_text = f"U[{ctx_spec[0]},{ctx_spec[1]}] seed {seed}"
    else:
        ctx_len = [ctx_spec] * B
        ctx_text = str(ctx_spec)
    CTX = max(ctx_len)
    tokens0 = rng.integers(0, cfg.vocab_size, B).astype(np.uint32)   # identical on every rank
    nblk = [(c + K + W + BLOCK) // BLOCK + 1 for c in ctx_len]
    first = np.concatenate([[0], np.cumsum(nblk)]).astype(int)
    tables = [list(range(int(first[b]), int(first[b + 1]))) for b in range(B)]

    def barrier(group_world):
        torch.cuda.synchronize()
        if group_world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(tp: int, nccl_exchange: bool):
        ident = exchange_unique_id(api.nccl_unique_id, dist) if tp > 1 else None
        tstream = torch.cuda.Stream()
        torch.cuda.set_stream(tstream)
        ctx = api.Context(local_rank, stream=tstream.cuda_stream, rank=rank if tp > 1 else 0, tp=tp, nccl_id=ident)
        if args.attn_grid:
            ctx.set_option(api._lib.PI_OPT_ATTN_FLAT, 0)
        exchange = "single GPU"
        if tp > 1:
            exchange = "nccl all-reduce"
            if not nccl_exchange:
                enable_peer_exchange(ctx, B * cfg.hidden_size, dist)
                exchange = "peer memory: partial sums pushed from the projection's epilogue (peer stores), flags, residual add folded in"
                if args.tp_pull:
                    ctx.set_option(api._lib.PI_OPT_TP_PUSH, 0)
                    exchange = "peer memory: partial sums fetched by the exchange kernel (P2P loads), flags, residual add folded in"
        model = api.LlamaWeights.synthetic(ctx, cfg, seed=seed, std=0.02, max_batch=B, max_positions=CTX + K + W + 8)
        kv = api.KvCache(ctx, model.kv_layout(int(first[-1]), BLOCK))
        kv.fill_normal(77 + (rank if tp > 1 else 0), 1.0)
        pos = list(ctx_len)
        out = model.decode_multi(tokens0, pos, tables, kv, W)
        tokens, pos = out[-1].copy(), [p + W for p in pos]
        sampler = ClockSampler(local_rank)
        sampler.start()
        time.sleep(0.3)
        barrier(tp)
        ctx.reset_kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        out = model.decode_multi(tokens, pos, tables, kv, K)
        e1.record()
        barrier(tp)
        t1 = time.time()
        launches = ctx.kernel_launches()
        clocks = sampler.stop(t0, t1)
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if tp > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        ms = float(ms[0])
        # one profiled pass for the per-class shares (this rank's view)
        ctx.profile_begin()
        model.decode_multi(out[-1].copy(), [p + K for p in pos], tables, kv, 2)
        prof = ctx.profile_end()
        total = sum(v[0] for v in prof.values()) or 1e-9
        weight_bytes = model.weight_bytes()                         # this rank's shard
        kv_bytes = sum(c + W + K // 2 for c in ctx_len) * (cfg.num_key_value_heads // tp) * 2 * cfg.head_dim * 4 * cfg.num_hidden_layers
        step_ms = ms / K
        res = {"tp": tp, "ms_per_step": round(step_ms, 4), "tok/s": round(B * K / (ms / 1e3), 1), "steps": K, "exchange": exchange,
               "collectives_per_step": 2 * cfg.num_hidden_layers + 1 if tp > 1 else 0, "gpu_launches": launches, "clocks": clocks,
               "step_roofline": {"bytes_per_step_per_gpu": weight_bytes + kv_bytes, "weight_bytes_per_gpu": weight_bytes,
                                 "kv_bytes_per_gpu": kv_bytes, "achieved_GB/s_per_gpu": round((weight_bytes + kv_bytes) / (step_ms / 1e3) / 1e9, 1),
                                 "peak_GB/s": hbm_peak, "frac": round((weight_bytes + kv_bytes) / (step_ms / 1e3) / 1e9 / hbm_peak, 3),
                                 "peak_kind": f"of {peak_kind}"},
               "device_time_shares": {c: round(v[0] / total, 3) for c, v in prof.items() if v[0] > 0}}
        if tp > 1:
            dist.barrier()       # peers read each other's buffers: nobody tears down before everyone is done
        kv.close()
        model.close()
        ctx.close()
        return res

    main = measure(world, args.nccl_exchange)
    tp1 = None
    if with_tp1 and world > 1:
        if rank == 0:
            tp1 = measure(1, False)
        dist.barrier()
    if rank != 0:
        return None
    out = {"metric": f"int8 batched paged decode throughput ({model_name} arch, batch {B}, context {ctx_text}, tensor parallel)",
           "workload": workload, "scaling": "strong", "batch": B, "context": ctx_text, "block_size": BLOCK,
           "weights": f"N(0,0.02) generated on device, seed {seed}", "kv": "N(0,1) fill"}
    out.update(main)
    if tp1 is not None:
        out["tp1"] = {k: tp1[k] for k in ("ms_per_step", "tok/s", "step_roofline", "device_time_shares")}
        out["speedup_over_tp1"] = round(tp1["ms_per_step"] / main["ms_per_step"], 3)
    return out


def run_tp_workload(args, rank: int, world: int, local_rank: int):
    """`--workload llama3_8b_tp`: Llama-3-8B architecture, int8 projections, batch 32 decode at context 4096;
    `--workload llama2_70b_tp`: Llama-2-70B architecture, batch 64, contexts U[1024,4096] (needs >= 2 GPUs).
    Tensor-parallel over all `world` ranks (strong scaling: the total work is fixed)."""
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    K, W = args.steps, max(args.warmup, 3)
    res = tp_decode(args, args.workload, rank, world, local_rank, K, W, with_tp1=False)
    if rank == 0:
        line = {
            "metric": res["metric"], "value": res["tok/s"], "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 weights, f32 activations/accumulate/KV", "data": "synthetic",
            "config": {"workload": args.workload, "batch": res["batch"], "context": res["context"], "block_size": BLOCK,
                       "parallelism": f"tp{world}", "collectives_per_step": res["collectives_per_step"], "exchange": res["exchange"],
                       "weights": res["weights"], "kv": res["kv"]},
            "gpu_launches": res["gpu_launches"], "clocks": res["clocks"], "step_roofline": res["step_roofline"],
            "device_time_shares": res["device_time_shares"],
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
    # a single attention call takes the flat tile list only on request (it pays for its own work-list kernel)
    ctx.set_option(api._lib.PI_OPT_ATTN_FLAT, 0 if args.attn_grid else 2)
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
        ctx.profile_begin()                      # device time of the launches only: packing the tables on the host is slow
        for r in range(reps):
            attn.run_device(qv, ov, kv, entries)
        prof = ctx.profile_end()
        us = prof["attention"][0] * 1e3 / reps   # all launches of one call (work list + kernel, or kernel + merge)
        algo = B * ctx_len * cfg.num_key_value_heads * 2 * cfg.head_dim * 4 + 2 * qv.numel() * 4
        print(json.dumps({"kernel_case": case, "calls": reps, "us_per_call": round(us, 2), "launches_per_call": prof["attention"][1] / reps,
                          "algorithmic_bytes": algo, "GB/s": round(algo / us / 1e3, 1),
                          "frac_of_hbm_peak": round(algo / us / 1e3 / measured_peaks()[0], 3), "peak_kind": f"of {measured_peaks()[2]}"}),
              flush=True)
        return
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
    hbm_peak, _, peak_kind = measured_peaks()
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
    ap.add_argument("--resident-only", action="store_true",
                    help="for a profiler's launch list: only the resident decode leg (warm-up + timed steps) over a pool filled with "
                         "N(0,1) values; prints its step time and exits")
    ap.add_argument("--nccl-exchange", action="store_true", help="tensor-parallel workloads: all-reduce through NCCL instead of the peer-memory kernels")
    ap.add_argument("--attn-grid", action="store_true",
                    help="batched decode attention on the per-entry grid (kv head, entry, KV split) instead of the flat tile list")
    ap.add_argument("--tp-pull", action="store_true", help="tensor-parallel workloads: the exchange kernel fetches the peers' partial sums (no push)")
    args = ap.parse_args()
    # stdout carries exactly one JSON line: whatever NCCL logs goes to stderr
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
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
