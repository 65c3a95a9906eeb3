"""The whole forward pass on the GPU, through the C ABI.

1. The reference's golden fixture (NumPy HF-Llama logits; F32 = bf16 checkpoint
   weights): tolerance 5e-4 and zero argmax mismatches, exactly the reference's
   own bar (tests/golden_parity_tests.rs:159-166, :208).
2. int8 projections against the oracle's int8 CPU path on the same weights:
   logits within 1e-3 max-abs and zero greedy-argmax mismatches (the bar the
   project states), batched == single within 1e-5, chunked prefill == sequential.
3. The KV pool contents after a forward equal the oracle's cache within 1e-5.
"""
import numpy as np
import pytest

from helpers import compare_logits, load_golden, normal_f32, oracle_model

pytestmark = pytest.mark.gpu
BLOCK = 16


@pytest.fixture(scope="module")
def ctx():
    from paged_infer_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def gpu_model(ctx, cfg, hw, quant="f32", lm_head_int8=False, max_batch=64):
    from paged_infer_b200 import api
    import copy
    cfg = copy.copy(cfg)
    cfg.quantization = quant
    return api.LlamaWeights(ctx, cfg, hw, max_batch=max_batch, lm_head_int8=lm_head_int8)


def kv_floats(cfg, blocks, bs=BLOCK):
    return cfg.num_hidden_layers * blocks * bs * cfg.num_key_value_heads * 2 * cfg.head_dim


def test_golden_incremental_decode(ctx, oracle):  # golden_parity_tests.rs:125-167
    from paged_infer_b200 import api
    cfg, tokens, golden, hw = load_golden()
    m = gpu_model(ctx, cfg, hw)
    kv = api.KvCache(ctx, m.kv_layout(5, BLOCK))
    table = api.BlockTable([4, 2, 3])  # scattered physical blocks
    got = np.stack([m.forward(int(t), i, table, kv) for i, t in enumerate(tokens)])
    max_abs, mism = compare_logits(got, golden, oracle.argmax)
    assert max_abs < 5e-4 and mism == 0, (max_abs, mism)


def test_golden_prefill_and_split_prefill(ctx, oracle):  # golden_parity_tests.rs:173-259
    from paged_infer_b200 import api
    cfg, tokens, golden, hw = load_golden()
    m = gpu_model(ctx, cfg, hw)
    table = api.BlockTable([0, 1, 2])
    ref = None
    for chunk in (1, 2, 4, 8, 16, 64):
        kv = api.KvCache(ctx, m.kv_layout(3, BLOCK))
        got, tok = m.prefill_batched(tokens, 0, table, kv, chunk, want_argmax=True)
        assert np.abs(got - golden[-1]).max() < 5e-4
        assert tok == oracle.argmax(golden[-1])
        ref = got if ref is None else ref
        assert np.abs(got - ref).max() < 1e-5, chunk        # batched_decode_tests.rs:342-373
    kv = api.KvCache(ctx, m.kv_layout(3, BLOCK))
    m.prefill(tokens[:23], 0, table, kv)
    split = m.prefill(tokens[23:], 23, table, kv)
    assert np.abs(split - ref).max() < 1e-5


def test_golden_interleaved_rope_is_a_different_model(ctx, oracle):
    import copy, os
    from helpers import GOLDEN
    from paged_infer_b200 import api
    cfg, tokens, golden, hw = load_golden()
    cfg2 = copy.copy(cfg)
    cfg2.rope_style = 1
    m = gpu_model(ctx, cfg2, hw)
    kv = api.KvCache(ctx, m.kv_layout(3, BLOCK))
    got = np.stack([m.forward(int(t), i, [0, 1, 2], kv) for i, t in enumerate(tokens)])
    inter = np.fromfile(os.path.join(GOLDEN, "tiny_llama_interleaved_golden.bin"), "<f4").reshape(golden.shape)
    assert np.abs(got - inter).max() < 5e-4
    assert np.abs(got - golden).max() > 1e-2


@pytest.mark.parametrize("quant,lm8", [("f32", False), ("int8", False), ("int8", True)])
def test_fixture_model_matches_oracle_and_kv_contents(ctx, oracle, quant, lm8):
    from paged_infer_b200 import api
    cfg, tokens, golden, hw = load_golden()
    om = oracle_model(oracle, cfg, hw, quant, lm8)
    gm = gpu_model(ctx, cfg, hw, quant, lm8)
    if quant == "int8" and lm8:  # same bytes as QuantizedLinear::weight_bytes (bf16 storage halves the f32 ones)
        assert gm.weight_bytes() == om.weight_bytes()
    blocks = 8
    okv = np.zeros(kv_floats(cfg, blocks), np.float32)
    gkv = api.KvCache(ctx, gm.kv_layout(blocks, BLOCK))
    gkv.upload(okv)
    table = [5, 1, 6]
    want = np.stack([om.forward(int(t), i, table, okv, BLOCK) for i, t in enumerate(tokens)])
    got = np.stack([gm.forward(int(t), i, table, gkv) for i, t in enumerate(tokens)])
    max_abs, mism = compare_logits(got, want, oracle.argmax)
    assert max_abs < 1e-4 and mism == 0, (max_abs, mism)
    assert np.abs(gkv.download() - okv).max() < 1e-5


def test_batched_decode_equals_single_sequence(ctx, oracle):  # batched_decode_tests.rs:158-263
    from paged_infer_b200 import api
    cfg, tokens, golden, hw = load_golden()
    for window in (None, 7):
        import copy
        c = copy.copy(cfg)
        c.attention_window = window
        om = oracle_model(oracle, c, hw, "int8")
        gm = gpu_model(ctx, c, hw, "int8")
        lens = [5, 17, 16, 30, 1, 31, 32]
        tables = [[3 * b + i for i in range(3)] for b in range(len(lens))]
        okv = np.zeros(kv_floats(cfg, 3 * len(lens)), np.float32)
        gkv_b = api.KvCache(ctx, gm.kv_layout(3 * len(lens), BLOCK))
        gkv_s = api.KvCache(ctx, gm.kv_layout(3 * len(lens), BLOCK))
        gkv_b.upload(okv)  # the pool starts undefined; the oracle's cache starts at zero
        for b, n in enumerate(lens):
            om.prefill(tokens[:n], 0, tables[b], okv, BLOCK)
            gm.prefill_batched(tokens[:n], 0, tables[b], gkv_b, 8)
            gm.prefill_batched(tokens[:n], 0, tables[b], gkv_s, 8)
        nxt = [int(tokens[n]) for n in lens]
        got, ids = gm.decode_batch_into(nxt, lens, tables, gkv_b, want_argmax=True)
        want = om.decode_batch(nxt, lens, tables, okv, BLOCK)
        assert np.abs(got - want).max() < 1e-4
        assert ids.tolist() == [oracle.argmax(r) for r in want]
        for b, n in enumerate(lens):
            solo = gm.forward(nxt[b], n, tables[b], gkv_s)
            assert np.abs(got[b] - solo).max() < 1e-5, b
        assert np.abs(gkv_b.download() - okv).max() < 1e-5


def test_prefill_resume_causality_and_unmapped_write(ctx, oracle):  # batched_decode_tests.rs:375-492
    from paged_infer_b200 import api
    cfg, tokens, golden, hw = load_golden()
    om = oracle_model(oracle, cfg, hw, "int8")
    gm = gpu_model(ctx, cfg, hw, "int8")
    table = [2, 0, 1]
    # resume mid-prompt with a chunk size that does not divide the remainder, larger than the capacity clamp
    okv = np.zeros(kv_floats(cfg, 3), np.float32)
    gkv = api.KvCache(ctx, gm.kv_layout(3, BLOCK))
    gkv.upload(okv)
    om.prefill_batched(tokens[:11], 0, table, okv, BLOCK, 4)
    gm.prefill_batched(tokens[:11], 0, table, gkv, 4)
    want = om.prefill_batched(tokens[11:], 11, table, okv, BLOCK, 7)
    got = gm.prefill_batched(tokens[11:], 11, table, gkv, 7)
    assert np.abs(got - want).max() < 1e-4
    assert np.abs(gm.prefill_batched(tokens[11:], 11, table, gkv, 1000) - want).max() < 1e-4
    # causality: changing a LATER token of the chunk must not change an earlier position's KV
    before = gkv.download()
    t2 = tokens.copy()
    t2[39] = (t2[39] + 1) % cfg.vocab_size
    gm.prefill_batched(t2, 0, table, gkv, 64)
    after = gkv.download()
    L = api.KvLayout(cfg.num_hidden_layers, 3, BLOCK, cfg.num_key_value_heads, cfg.head_dim)
    i38 = L.index(1, table[2], 38 - 32, 0, False)
    assert np.abs(after[i38:i38 + cfg.head_dim] - before[i38:i38 + cfg.head_dim]).max() < 1e-6
    # a position past the mapped blocks: the K/V write is skipped silently, logits still come back
    short = [2, 0]
    okv2, gkv2 = np.zeros(kv_floats(cfg, 3), np.float32), api.KvCache(ctx, gm.kv_layout(3, BLOCK))
    gkv2.upload(okv2)
    want = om.prefill_batched(tokens[:36], 0, short, okv2, BLOCK, 8)
    got = gm.prefill_batched(tokens[:36], 0, short, gkv2, 8)
    assert np.all(np.isfinite(got)) and np.abs(got - want).max() < 1e-4
    assert np.abs(gkv2.download() - okv2).max() < 1e-5


def test_errors_match_the_reference_assertions(ctx):
    from paged_infer_b200 import api
    cfg, tokens, golden, hw = load_golden()
    gm = gpu_model(ctx, cfg, hw, "int8", max_batch=4)
    kv = api.KvCache(ctx, gm.kv_layout(3, BLOCK))
    with pytest.raises(api.PiError, match="exceeds scratch capacity"):
        gm.decode_batch_into([1] * 5, [0] * 5, [[0]] * 5, kv)
    with pytest.raises(api.PiError, match="at least one"):
        gm.decode_batch_into([], [], [], kv)
    with pytest.raises(api.PiError, match="at least one token"):
        gm.prefill_batched([], 0, [0], kv, 4)
    wrong = api.KvCache(ctx, api.KvLayout(cfg.num_hidden_layers, 3, BLOCK, cfg.num_key_value_heads + 1, cfg.head_dim))
    with pytest.raises(api.PiError, match="does not match"):
        gm.forward(1, 0, [0], wrong)
    assert np.all(np.isfinite(gm.forward(1, 0, [0], kv)))


def small_llama(ctx, oracle, seed, layers=2, hidden=512, heads=8, kv_heads=2, inter=1408, vocab=1000):
    """A TinyLlama-proportioned model (head_dim 64, kv_group 4, SwiGLU) small enough for the CPU oracle."""
    from paged_infer_b200 import api
    from paged_infer_b200.loader import HostWeights, LlamaConfig, f32_to_bf16_bits
    cfg = LlamaConfig(hidden, layers, heads, kv_heads, inter, vocab, 1e-5, 10000.0, quantization="int8")
    hd = hidden // heads
    shapes = {"wq": (hidden, hidden), "wk": (kv_heads * hd, hidden), "wv": (kv_heads * hd, hidden),
              "wo": (hidden, hidden), "w1": (inter, hidden), "w2": (hidden, inter), "w3": (inter, hidden)}
    projs = []
    for l in range(layers):
        d = {}
        for j, (k, shp) in enumerate(shapes.items()):
            w = normal_f32(shp, seed * 1000 + l * 10 + j, 0.02)
            d[k] = oracle.quantize_rows_i8(w, *shp)
        projs.append(d)
    lm = oracle.quantize_rows_i8(normal_f32((vocab, hidden), seed * 1000 + 999, 0.02), vocab, hidden)
    hw = HostWeights(f32_to_bf16_bits(normal_f32((vocab, hidden), seed * 1000 + 998, 0.02)), np.ones(hidden, np.float32),
                     [np.ones(hidden, np.float32)] * layers, [np.ones(hidden, np.float32)] * layers, projs, None)
    om = oracle.Model(cfg.as_dict(), hw.token_embeddings, hw.final_norm, hw.attention_norm, hw.ffn_norm, projs, lm)
    gm = api.LlamaWeights(ctx, cfg, hw, max_batch=64, lm_head=lm)
    return cfg, om, gm


def test_head_dim_64_model_prefill_then_greedy_decode(ctx, oracle):
    """Scaled-down config 0: prefill 128 random ids, then 128 teacher-forced greedy steps; 1e-3 / zero mismatches."""
    from paged_infer_b200 import api
    cfg, om, gm = small_llama(ctx, oracle, 0)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab_size, 128).astype(np.uint32)
    nblocks = 16
    table = list(rng.permutation(nblocks + 4)[:nblocks])
    okv = np.zeros(kv_floats(cfg, nblocks + 4), np.float32)
    gkv = api.KvCache(ctx, gm.kv_layout(nblocks + 4, BLOCK))
    gkv.upload(okv)
    want = om.prefill_batched(prompt, 0, table, okv, BLOCK, 32)
    got, tok = gm.prefill_batched(prompt, 0, table, gkv, 32, want_argmax=True)
    worst = np.abs(got - want).max()
    mism = int(tok != oracle.argmax(want))
    nxt = oracle.argmax(want)
    for step in range(128):
        pos = 128 + step
        want = om.forward(nxt, pos, table, okv, BLOCK)
        got, ids = gm.decode_batch_into([nxt], [pos], [table], gkv, want_argmax=True)
        worst = max(worst, np.abs(got[0] - want).max())
        mism += int(ids[0] != oracle.argmax(want))
        nxt = oracle.argmax(want)  # teacher forcing: one flip cannot cascade
    assert worst < 1e-3 and mism == 0, (worst, mism)
    assert np.abs(gkv.download() - okv).max() < 1e-4


def test_batch_64_ragged_decode_with_shared_prefix_blocks(ctx, oracle):
    """Scaled-down config 2: 64 sequences, ragged contexts, half of them sharing the
    physical blocks of a common prefix, several steps."""
    from paged_infer_b200 import api
    cfg, om, gm = small_llama(ctx, oracle, 2)
    rng = np.random.default_rng(2)
    B, prefix_blocks = 64, 2
    ctxlen = rng.integers(40, 120, B)
    total_blocks = 2 + B * 8
    free = list(range(total_blocks))[::-1]
    shared = [free.pop() for _ in range(prefix_blocks)]
    tables, seqs = [], []
    okv = np.zeros(kv_floats(cfg, total_blocks), np.float32)
    gkv = api.KvCache(ctx, gm.kv_layout(total_blocks, BLOCK))
    prefix = rng.integers(0, cfg.vocab_size, prefix_blocks * BLOCK).astype(np.uint32)
    for b in range(B):
        n = int(ctxlen[b])
        own = [free.pop() for _ in range(8 - (prefix_blocks if b < B // 2 else 0))]
        if b < B // 2:
            tables.append(shared + own)
            seqs.append(np.concatenate([prefix, rng.integers(0, cfg.vocab_size, n - prefix.size).astype(np.uint32)]))
        else:
            tables.append(own)
            seqs.append(rng.integers(0, cfg.vocab_size, n).astype(np.uint32))
    # the shared prefix is computed once (sequence 0); everyone else resumes after it, like a prefix-cache hit
    for b in range(B):
        start = 0 if (b == 0 or b >= B // 2) else prefix.size
        om.prefill_batched(seqs[b][start:], start, tables[b], okv, BLOCK, 32)
    gkv.upload(okv)
    nxt = [int(rng.integers(0, cfg.vocab_size)) for _ in range(B)]
    pos = [int(n) for n in ctxlen]
    worst, mism = 0.0, 0
    for step in range(3):
        want = om.decode_batch(nxt, pos, tables, okv, BLOCK)
        got, ids = gm.decode_batch_into(nxt, pos, tables, gkv, want_argmax=True)
        worst = max(worst, np.abs(got - want).max())
        wa = [oracle.argmax(r) for r in want]
        mism += sum(int(a != b) for a, b in zip(ids.tolist(), wa))
        nxt, pos = wa, [p + 1 for p in pos]
    assert worst < 1e-3 and mism == 0, (worst, mism)


def test_logits_of_selected_rows_only(ctx, oracle):
    """The per-sequence hand-off of Engine::run_groups (src/engine.rs:742-755): ids for everyone, full logits only for
    the rows the host samples itself."""
    from paged_infer_b200 import api
    cfg, om, gm = small_llama(ctx, oracle, 6)
    rng = np.random.default_rng(6)
    B = 9
    lens = [int(x) for x in rng.integers(3, 40, B)]
    tables = [[b * 4 + i for i in range(4)] for b in range(B)]
    kv = api.KvCache(ctx, gm.kv_layout(4 * B, BLOCK))
    kv.upload(np.zeros(kv_floats(cfg, 4 * B), np.float32))
    for b in range(B):
        gm.prefill_batched(rng.integers(0, cfg.vocab_size, lens[b]).astype(np.uint32), 0, tables[b], kv, 16)
    tok = rng.integers(0, cfg.vocab_size, B).astype(np.uint32)
    full, ids = gm.decode_batch_into(tok, lens, tables, kv, want_argmax=True)
    some, ids2 = gm.decode_batch_rows(tok, lens, tables, kv, [7, 0, 3])      # same step again: same KV values rewritten
    assert ids2.tolist() == ids.tolist()
    assert np.array_equal(some, full[[7, 0, 3]])
    none, ids3 = gm.decode_batch_rows(tok, lens, tables, kv, [])
    assert none.shape == (0, cfg.vocab_size) and ids3.tolist() == ids.tolist()
    with pytest.raises(api.PiError, match="row 9"):
        gm.decode_batch_rows(tok, lens, tables, kv, [9])


def test_multi_step_decode_equals_step_by_step(ctx, oracle):
    """n greedy steps in one call (eager first step, then a replayed CUDA graph) == n single-step calls."""
    from paged_infer_b200 import api
    cfg, om, gm = small_llama(ctx, oracle, 5)
    rng = np.random.default_rng(5)
    for B, n in ((1, 9), (7, 6), (40, 5), (3, 2)):
        lens = [int(x) for x in rng.integers(3, 60, B)]
        tables = [[b * 6 + i for i in range(6)] for b in range(B)]
        kv_a = api.KvCache(ctx, gm.kv_layout(6 * B, BLOCK))
        kv_b = api.KvCache(ctx, gm.kv_layout(6 * B, BLOCK))
        zero = np.zeros(kv_floats(cfg, 6 * B), np.float32)
        kv_a.upload(zero)
        kv_b.upload(zero)
        for b in range(B):
            prompt = rng.integers(0, cfg.vocab_size, lens[b]).astype(np.uint32)
            gm.prefill_batched(prompt, 0, tables[b], kv_a, 16)
            gm.prefill_batched(prompt, 0, tables[b], kv_b, 16)
        tok = rng.integers(0, cfg.vocab_size, B).astype(np.uint32)
        multi = gm.decode_multi(tok, lens, tables, kv_a, n)
        cur, pos = tok, list(lens)
        for s in range(n):
            cur = gm.decode_batch_into(cur, pos, tables, kv_b, want_logits=False, want_argmax=True)
            assert multi[s].tolist() == cur.tolist(), (B, s)
            pos = [p + 1 for p in pos]
        assert np.abs(kv_a.download() - kv_b.download()).max() < 1e-5


def test_multi_step_decode_over_the_flat_work_list(ctx, oracle):
    """A batch with enough K|V tiles for the flat attention work list (64 sequences of 600-700 tokens): the work list is
    rebuilt on the device from the positions every step, so n steps inside one call (CUDA graph, positions advanced on
    the device, blocks crossed on the way) must give the ids and the KV of n single-step calls; the
    per-entry grid (option off) must agree on the logits to rounding."""
    from paged_infer_b200 import _lib, api
    cfg, om, gm = small_llama(ctx, oracle, 8)
    rng = np.random.default_rng(8)
    B, n, nblk = 64, 20, 46
    pos0 = [int(x) for x in rng.integers(600, 700, B)]
    tables = [[int(t) for t in rng.permutation(nblk) + b * nblk] for b in range(B)]
    caches = []
    for _ in range(3):
        kv = api.KvCache(ctx, gm.kv_layout(nblk * B, BLOCK))
        kv.fill_normal(3, 1.0)
        caches.append(kv)
    tok = rng.integers(0, cfg.vocab_size, B).astype(np.uint32)
    launches0 = ctx.kernel_launches()
    multi = gm.decode_multi(tok, pos0, tables, caches[0], n)
    per_step = (ctx.kernel_launches() - launches0) / n
    cur, pos = tok, list(pos0)
    for s in range(n):
        cur = gm.decode_batch_into(cur, pos, tables, caches[1], want_logits=False, want_argmax=True)
        assert multi[s].tolist() == cur.tolist(), s
        pos = [p + 1 for p in pos]
    assert np.abs(caches[0].download() - caches[1].download()).max() < 1e-6
    # one launch per layer for the attention (no merge launch) + the work list: 5 per layer + embed, planes, LM head, argmax, advance
    assert per_step <= 5 * cfg.num_hidden_layers + 7, per_step
    flat_logits, _ = gm.decode_batch_into(tok, pos0, tables, caches[2], want_argmax=True)
    ctx.set_option(_lib.PI_OPT_ATTN_FLAT, 0)
    try:
        grid_logits, _ = gm.decode_batch_into(tok, pos0, tables, caches[2], want_argmax=True)
    finally:
        ctx.set_option(_lib.PI_OPT_ATTN_FLAT, 1)
    assert np.abs(flat_logits - grid_logits).max() < 1e-4
    assert not np.array_equal(flat_logits, grid_logits), "the flat work list was not used"
