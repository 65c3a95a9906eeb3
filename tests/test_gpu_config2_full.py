"""The benchmarked batch at its real geometry: 64 sequences at TinyLlama width (hidden 2048, 32 query / 4 KV heads
of 64, FFN 5632, vocab 32000, int8 LM head), contexts uniform in [256, 2048] from seed 2, KV block size 16,
sequences 0-31 mapping the SAME physical blocks for a common 512-token prefix, sequences 56-63 forked from 48-55
(same table, partial last block shared) with the copy-on-write split on the first write after the fork.

The KV is produced by prefill on both sides (the CUDA library and the CPU oracle, each into its own pool), then
teacher-forced batched decode steps are compared with the oracle's int8 CPU path: logits within 1e-3, zero greedy
mismatches, and the pools agree afterwards.  Four layers instead of 22 keep the CPU side to a minute or two; the
width, the context lengths, head_dim 64, the KV-split attention with its merge kernel emitting planes, the
tensor-core projections handing planes to each other and the 32-block shared prefix are the benchmark's.

Block bookkeeping follows the reference engine: prefix hit on full blocks only (src/memory/kv_cache_manager.rs:
116-200), fork = table copy with the reference counts bumped (:262-296), ensure_writable before the step's forward
(:298-327, src/engine.rs:670-676).
"""
import numpy as np
import pytest

from test_gpu_config_shapes import kv_floats, wide_llama

pytestmark = pytest.mark.gpu
BLOCK = 16


class Blocks:
    """Reference-counted physical blocks + per-sequence tables (host side of the engine for this batch)."""

    def __init__(self, total):
        self.free = list(range(total))[::-1]
        self.ref = [0] * total
        self.cow = 0

    def alloc(self):
        b = self.free.pop()
        self.ref[b] = 1
        return b

    def ensure_writable(self, table, pos, copy):
        lb = pos // BLOCK
        if lb >= len(table):
            table.append(self.alloc())
        elif self.ref[table[lb]] > 1:
            dst = self.alloc()
            copy(table[lb], dst)
            self.ref[table[lb]] -= 1
            table[lb] = dst
            self.cow += 1


@pytest.fixture(scope="module")
def ctx():
    from paged_infer_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def test_config2_geometry_prefix_sharing_cow_forks(ctx, oracle):
    from paged_infer_b200 import api
    layers, B, forks, prefix_tokens, steps, multi_steps = 4, 64, 8, 512, 4, 5
    cfg, om, gm = wide_llama(ctx, oracle, 31, hidden=2048, heads=32, kv_heads=4, inter=5632, vocab=32000, theta=10000.0,
                             layers=layers, max_batch=512)
    rng = np.random.default_rng(2)
    lens = rng.integers(256, 2049, B)
    lens[B - forks:] = lens[B - 2 * forks:B - forks]          # a fork starts at its parent's length
    lens = [int(n) for n in lens]
    total_blocks = sum((n + steps + multi_steps) // BLOCK + 2 for n in lens) + 16
    blocks = Blocks(total_blocks)
    okv = np.zeros(kv_floats(cfg, total_blocks), np.float32)
    gkv = api.KvCache(ctx, gm.kv_layout(total_blocks, BLOCK))
    gkv.upload(okv)
    olayout = oracle.kv_layout(layers, total_blocks, BLOCK, cfg.num_key_value_heads, cfg.head_dim)

    prefix = rng.integers(0, cfg.vocab_size, prefix_tokens).astype(np.uint32)
    shared, computed_shared = [], 0
    tables = []
    worst = 0.0
    for b in range(B - forks):
        n = lens[b]
        t = []
        start = 0
        if b < B // 2:                                         # prefix-cache hit on whole blocks
            n_shared = min(prefix_tokens // BLOCK, n // BLOCK)
            while len(shared) < n_shared:
                shared.append(blocks.alloc())
            for pb in shared[:n_shared]:
                blocks.ref[pb] += 1
                t.append(pb)
            tokens = np.concatenate([prefix, rng.integers(0, cfg.vocab_size, max(n - prefix_tokens, 0)).astype(np.uint32)])[:n]
            # resume behind the shared blocks that an earlier sequence has already filled; a prompt that is cached
            # in full recomputes its last token into the shared block (src/engine.rs:509-512)
            start = min(min(n_shared, computed_shared) * BLOCK, n - 1)
            computed_shared = max(computed_shared, n_shared)
        else:
            tokens = rng.integers(0, cfg.vocab_size, n).astype(np.uint32)
        while len(t) < (n + BLOCK - 1) // BLOCK:
            t.append(blocks.alloc())
        tables.append(t)
        want = om.prefill_batched(tokens[start:], start, t, okv, BLOCK, 64)
        got = gm.prefill_batched(tokens[start:], start, t, gkv, 512 if b % 2 else 64)   # both chunked-attention kernels
        worst = max(worst, float(np.abs(got - want).max()))
    assert len(shared) == prefix_tokens // BLOCK
    assert worst < 1e-3, worst
    for b in range(B - forks, B):                              # fork: the parent's table, every block shared
        parent = tables[b - forks]
        for pb in parent:
            blocks.ref[pb] += 1
        tables.append(list(parent))
    assert float(np.abs(gkv.download() - okv).max()) < 1e-4

    def copy(src, dst):
        oracle.kv_copy_block(olayout, okv, src, dst)
        gkv.copy_block(src, dst)

    nxt = [int(t) for t in rng.integers(0, cfg.vocab_size, B)]   # forks continue with a token of their own
    pos = list(lens)
    mism = 0
    ctx.profile_begin()
    for step in range(steps):
        for b in range(B):
            blocks.ensure_writable(tables[b], pos[b], copy)
        if step == 0:
            assert blocks.cow == forks                           # one split per parent/child pair, on the first write
            assert all(tables[b][-1] != tables[b - forks][-1] for b in range(B - forks, B))
            assert all(tables[b][:32] == shared for b in range(B // 2) if lens[b] >= prefix_tokens)
        want = om.decode_batch(nxt, pos, tables, okv, BLOCK)
        got, ids = gm.decode_batch_into(nxt, pos, tables, gkv, want_argmax=True)
        worst = max(worst, float(np.abs(got - want).max()))
        wa = [oracle.argmax(r) for r in want]
        mism += sum(int(a != w) for a, w in zip(ids.tolist(), wa))
        nxt, pos = wa, [p + 1 for p in pos]
    prof = ctx.profile_end()
    assert worst < 1e-3 and mism == 0, (worst, mism)
    assert prof["gemm_tc"][1] > 0 and prof["gemv"][1] == 0 and prof["attention"][1] >= steps * layers

    # the resident multi-step call (device-side position advance, CUDA graph replay) against the oracle running free
    for s in range(multi_steps):
        for b in range(B):
            blocks.ensure_writable(tables[b], pos[b] + s, copy)
    multi = gm.decode_multi(nxt, pos, tables, gkv, multi_steps)
    for s in range(multi_steps):
        want = om.decode_batch(nxt, pos, tables, okv, BLOCK)
        nxt = [oracle.argmax(r) for r in want]
        assert multi[s].tolist() == nxt, s
        pos = [p + 1 for p in pos]
    assert float(np.abs(gkv.download() - okv).max()) < 1e-4
    gkv.close()
