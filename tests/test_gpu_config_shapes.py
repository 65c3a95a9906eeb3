"""Parity at the real shapes of the benchmark configurations (one layer deep, so the CPU oracle stays quick):

* the GEMV / GEMM sweep over the TinyLlama projection shapes at 1, 8, 32, 128 and 512 activation rows;
* Llama-3-8B and Llama-2-70B projection shapes (K up to 28672, head_dim 128);
* full-width one-layer models (TinyLlama: hidden 2048, 32/4 heads, FF 5632, vocab 32000 with an int8 LM head;
  Llama-3-8B: hidden 4096, 32/8 heads of 128, FF 14336) with random RMSNorm weights, through chunked prefill,
  single-sequence decode (CUDA-core path) and batched decode (tensor-core path, where each projection hands its
  result to the next as bf16 planes): logits within 1e-3 of the oracle's int8 CPU path, zero greedy mismatches.
"""
import numpy as np
import pytest

from helpers import normal_f32

pytestmark = pytest.mark.gpu
BLOCK = 16


@pytest.fixture(scope="module")
def ctx():
    from paged_infer_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def rel_err(got, want):
    return float((np.abs(got - want) / np.maximum(np.abs(want), 1.0)).max())


@pytest.mark.parametrize("rows,cols", [(2048, 2048), (256, 2048), (5632, 2048), (2048, 5632)])
def test_projection_sweep_over_activation_rows(ctx, oracle, rows, cols):
    from paged_infer_b200 import api
    q, s = oracle.quantize_rows_i8(normal_f32((rows, cols), 11 + rows + cols, 0.02), rows, cols)
    p = api.Projection.int8(ctx, q, s)
    for M in (1, 8, 32, 128, 512):
        x = normal_f32((M, cols), 100 + M, 1.0)
        want = oracle.matmat_i8(x, q, s)
        got = p.apply_batched(x)
        assert rel_err(got, want) < 2e-5 * max(1.0, (cols / 2048.0) ** 0.5), (rows, cols, M)


def test_lm_head_shape(ctx, oracle):
    from paged_infer_b200 import api
    rows, cols = 32000, 2048
    q, s = oracle.quantize_rows_i8(normal_f32((rows, cols), 5, 0.02), rows, cols)
    p = api.Projection.int8(ctx, q, s)
    for M in (1, 8, 64, 128, 512):
        x = normal_f32((M, cols), 200 + M, 1.0)
        assert rel_err(p.apply_batched(x), oracle.matmat_i8(x, q, s)) < 2e-5, M


@pytest.mark.parametrize("rows,cols,M", [(4096, 4096, 32), (1024, 4096, 32), (4096, 14336, 32), (14336, 4096, 8),
                                         (8192, 8192, 64), (1024, 8192, 64), (2048, 28672, 16), (2048, 28672, 1)])
def test_llama3_and_llama2_70b_projection_shapes(ctx, oracle, rows, cols, M):
    from paged_infer_b200 import api
    q, s = oracle.quantize_rows_i8(normal_f32((rows, cols), rows * 3 + cols, 0.02), rows, cols)
    p = api.Projection.int8(ctx, q, s)
    x = normal_f32((M, cols), 300 + M, 1.0)
    assert rel_err(p.apply_batched(x), oracle.matmat_i8(x, q, s)) < 2e-5 * (cols / 2048.0) ** 0.5


def wide_llama(ctx, oracle, seed, hidden, heads, kv_heads, inter, vocab, theta, layers=1, max_batch=64, rope_style=0):
    """A full-width model with random RMSNorm weights (N(1, 0.2)) and an int8 LM head."""
    from paged_infer_b200 import api
    from paged_infer_b200.loader import HostWeights, LlamaConfig, f32_to_bf16_bits
    cfg = LlamaConfig(hidden, layers, heads, kv_heads, inter, vocab, 1e-5, theta, quantization="int8")
    cfg.rope_style = rope_style
    hd = hidden // heads
    shapes = {"wq": (hidden, hidden), "wk": (kv_heads * hd, hidden), "wv": (kv_heads * hd, hidden),
              "wo": (hidden, hidden), "w1": (inter, hidden), "w2": (hidden, inter), "w3": (inter, hidden)}
    projs = []
    for l in range(layers):
        projs.append({k: oracle.quantize_rows_i8(normal_f32(shp, seed * 1000 + l * 10 + j, 0.02), *shp)
                      for j, (k, shp) in enumerate(shapes.items())})
    lm = oracle.quantize_rows_i8(normal_f32((vocab, hidden), seed * 1000 + 999, 0.02), vocab, hidden)

    def norm(i):
        return (1.0 + normal_f32((hidden,), seed * 1000 + 900 + i, 0.2)).astype(np.float32)

    hw = HostWeights(f32_to_bf16_bits(normal_f32((vocab, hidden), seed * 1000 + 998, 0.5)), norm(0),
                     [norm(1 + l) for l in range(layers)], [norm(50 + l) for l in range(layers)], projs, None)
    om = oracle.Model(cfg.as_dict(), hw.token_embeddings, hw.final_norm, hw.attention_norm, hw.ffn_norm, projs, lm)
    gm = api.LlamaWeights(ctx, cfg, hw, max_batch=max_batch, lm_head=lm)
    return cfg, om, gm


def kv_floats(cfg, blocks):
    return cfg.num_hidden_layers * blocks * BLOCK * cfg.num_key_value_heads * 2 * cfg.head_dim


def run_model_case(ctx, oracle, cfg, om, gm, prompt_len, batch):
    from paged_infer_b200 import api
    rng = np.random.default_rng(9)
    blocks_per_seq = (prompt_len + 16) // BLOCK + 1
    nblocks = blocks_per_seq * (batch + 1)
    okv = np.zeros(kv_floats(cfg, nblocks), np.float32)
    gkv = api.KvCache(ctx, gm.kv_layout(nblocks, BLOCK))
    gkv.upload(okv)
    perm = rng.permutation(nblocks)
    tables = [[int(b) for b in perm[i * blocks_per_seq:(i + 1) * blocks_per_seq]] for i in range(batch + 1)]
    worst, mism = 0.0, 0

    # chunked prefill of sequence 0 (tensor-core path for the chunks), then single-sequence decode (CUDA-core path)
    prompt = rng.integers(0, cfg.vocab_size, prompt_len).astype(np.uint32)
    want = om.prefill_batched(prompt, 0, tables[0], okv, BLOCK, 32)
    got, tok = gm.prefill_batched(prompt, 0, tables[0], gkv, 32, want_argmax=True)
    worst = max(worst, float(np.abs(got - want).max()))
    mism += int(tok != oracle.argmax(want))
    nxt = oracle.argmax(want)
    for step in range(3):
        pos = prompt_len + step
        want = om.forward(nxt, pos, tables[0], okv, BLOCK)
        got, ids = gm.decode_batch_into([nxt], [pos], [tables[0]], gkv, want_argmax=True)
        worst = max(worst, float(np.abs(got[0] - want).max()))
        mism += int(ids[0] != oracle.argmax(want))
        nxt = oracle.argmax(want)

    # batched decode of `batch` other sequences with ragged contexts (tensor-core path, fused plane hand-off)
    lens = rng.integers(prompt_len // 2, prompt_len, batch)
    for b in range(batch):
        om.prefill_batched(rng.integers(0, cfg.vocab_size, int(lens[b])).astype(np.uint32), 0, tables[b + 1], okv, BLOCK, 32)
    gkv.upload(okv)
    toks = [int(t) for t in rng.integers(0, cfg.vocab_size, batch)]
    pos = [int(n) for n in lens]
    for step in range(2):
        want = om.decode_batch(toks, pos, tables[1:], okv, BLOCK)
        got, ids = gm.decode_batch_into(toks, pos, tables[1:], gkv, want_argmax=True)
        worst = max(worst, float(np.abs(got - want).max()))
        wa = [oracle.argmax(r) for r in want]
        mism += sum(int(a != b) for a, b in zip(ids.tolist(), wa))
        toks, pos = wa, [p + 1 for p in pos]
    return worst, mism


@pytest.mark.parametrize("batch", [24, 64])
def test_tinyllama_width_one_layer(ctx, oracle, batch):
    cfg, om, gm = wide_llama(ctx, oracle, 21, hidden=2048, heads=32, kv_heads=4, inter=5632, vocab=32000, theta=10000.0)
    worst, mism = run_model_case(ctx, oracle, cfg, om, gm, prompt_len=48, batch=batch)
    assert worst < 1e-3 and mism == 0, (worst, mism)


def test_llama3_8b_width_one_layer(ctx, oracle):
    cfg, om, gm = wide_llama(ctx, oracle, 22, hidden=4096, heads=32, kv_heads=8, inter=14336, vocab=4096, theta=500000.0,
                             max_batch=32)
    worst, mism = run_model_case(ctx, oracle, cfg, om, gm, prompt_len=40, batch=32)
    assert worst < 1e-3 and mism == 0, (worst, mism)


@pytest.mark.parametrize("heads,kv_heads,style", [(16, 4, 1), (8, 2, 0), (8, 2, 1)])
def test_rope_and_kv_write_in_the_projection_epilogue(ctx, oracle, heads, kv_heads, style):
    """Batched decode folds the rotary embedding and the KV write into the q/k/v projection: both pairing styles,
    head_dim 64 and 128, logits and the pool contents against the oracle."""
    from paged_infer_b200 import api
    cfg, om, gm = wide_llama(ctx, oracle, 31 + style, hidden=1024, heads=heads, kv_heads=kv_heads, inter=2816, vocab=2048,
                             theta=10000.0, layers=2, rope_style=style)
    rng = np.random.default_rng(5)
    B, nblocks = 40, 48
    okv = (rng.standard_normal(kv_floats(cfg, nblocks)) * 0.5).astype(np.float32)
    gkv = api.KvCache(ctx, gm.kv_layout(nblocks, BLOCK))
    gkv.upload(okv)
    tables = [[b] for b in range(B)]
    toks = [int(t) for t in rng.integers(0, cfg.vocab_size, B)]
    pos = [int(p) for p in rng.integers(0, BLOCK, B)]
    want = om.decode_batch(toks, pos, tables, okv, BLOCK)
    got = gm.decode_batch_into(toks, pos, tables, gkv, want_logits=True)
    assert np.abs(got - want).max() < 1e-3
    assert np.abs(gkv.download() - okv).max() < 1e-4


def test_two_layers_hand_planes_across_the_layer_boundary(ctx, oracle):
    """down -> next layer's q/k/v also goes through the plane hand-off (with the next layer's norm weight)."""
    cfg, om, gm = wide_llama(ctx, oracle, 23, hidden=1024, heads=16, kv_heads=4, inter=2816, vocab=2048, theta=10000.0, layers=3)
    worst, mism = run_model_case(ctx, oracle, cfg, om, gm, prompt_len=40, batch=48)
    assert worst < 1e-3 and mism == 0, (worst, mism)
    # and the fused hand-off agrees with the split-kernel path on the same inputs
    from paged_infer_b200 import api
    rng = np.random.default_rng(3)
    gkv = api.KvCache(ctx, gm.kv_layout(64, BLOCK))
    gkv.fill_normal(4, 1.0)
    toks = rng.integers(0, cfg.vocab_size, 48).astype(np.uint32)
    tables = [[b] for b in range(48)]
    fused = gm.decode_batch_into(toks, [7] * 48, tables, gkv, want_logits=True)
    ctx.set_option(api._lib.PI_OPT_FUSE_PLANES, 0)
    try:
        plain = gm.decode_batch_into(toks, [7] * 48, tables, gkv, want_logits=True)
    finally:
        ctx.set_option(api._lib.PI_OPT_FUSE_PLANES, 1)
    assert np.abs(fused - plain).max() < 1e-4


@pytest.mark.parametrize("arch", ["tinyllama", "llama3"])
def test_large_prefill_chunks_use_the_shared_table_attention(ctx, oracle, arch):
    """Prefill in chunks of 256 positions: the chunk's attention runs in the shared-table kernel (all positions of a
    chunk map one table); logits of the last position and the KV written on the way against the oracle."""
    from paged_infer_b200 import api
    if arch == "tinyllama":
        cfg, om, gm = wide_llama(ctx, oracle, 41, hidden=2048, heads=32, kv_heads=4, inter=5632, vocab=32000, theta=10000.0,
                                 max_batch=256)
    else:
        cfg, om, gm = wide_llama(ctx, oracle, 42, hidden=4096, heads=32, kv_heads=8, inter=14336, vocab=4096, theta=500000.0,
                                 max_batch=256)
    n, nblocks = 300, 24
    rng = np.random.default_rng(17)
    prompt = rng.integers(0, cfg.vocab_size, n).astype(np.uint32)
    table = [int(b) for b in rng.permutation(nblocks)[:n // BLOCK + 1]]
    okv = np.zeros(kv_floats(cfg, nblocks), np.float32)
    want = om.prefill_batched(prompt, 0, table, okv, BLOCK, 32)
    gkv = api.KvCache(ctx, gm.kv_layout(nblocks, BLOCK))
    gkv.upload(np.zeros_like(okv))
    ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, 2)
    try:
        got, tok = gm.prefill_batched(prompt, 0, table, gkv, 256, want_argmax=True)
    finally:
        ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, 1)
    assert np.abs(got - want).max() < 1e-3 and tok == oracle.argmax(want)
    assert np.abs(gkv.download() - okv).max() < 1e-4
    # and the same prompt through the per-entry decode kernel gives the same logits
    gkv.upload(np.zeros_like(okv))
    ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, 0)
    try:
        plain = gm.prefill_batched(prompt, 0, table, gkv, 256)
    finally:
        ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, 1)
    assert np.abs(got - plain).max() < 1e-4


def test_config0_full_size_prefill_128_then_128_greedy_steps(ctx, oracle):
    """The batch-1 benchmark configuration at FULL size: TinyLlama-1.1B architecture (22 layers, hidden 2048, 32/4 heads
    of 64, FFN 5632, vocab 32000), weights N(0, 0.02) quantised by the reference scheme, prompt of 128 uniform token
    ids, chunked prefill, then 128 greedy decode steps (teacher forced, so one flip could not cascade): logits within
    1e-3 of the oracle's int8 CPU path at every step and zero greedy mismatches."""
    from paged_infer_b200 import api
    cfg, om, gm = wide_llama(ctx, oracle, 0, hidden=2048, heads=32, kv_heads=4, inter=5632, vocab=32000, theta=10000.0,
                             layers=22, max_batch=32)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab_size, 128).astype(np.uint32)
    nblocks = 17
    table = [int(b) for b in rng.permutation(nblocks + 3)[:nblocks]]
    okv = np.zeros(kv_floats(cfg, nblocks + 3), np.float32)
    gkv = api.KvCache(ctx, gm.kv_layout(nblocks + 3, BLOCK))
    gkv.upload(okv)
    want = om.prefill_batched(prompt, 0, table, okv, BLOCK, 32)
    got, tok = gm.prefill_batched(prompt, 0, table, gkv, 32, want_argmax=True)
    worst = float(np.abs(got - want).max())
    mism = int(tok != oracle.argmax(want))
    nxt = oracle.argmax(want)
    for step in range(128):
        pos = 128 + step
        want = om.forward(nxt, pos, table, okv, BLOCK)
        got, ids = gm.decode_batch_into([nxt], [pos], [table], gkv, want_argmax=True)
        worst = max(worst, float(np.abs(got[0] - want).max()))
        mism += int(ids[0] != oracle.argmax(want))
        nxt = oracle.argmax(want)
    assert worst < 1e-3 and mism == 0, (worst, mism)
