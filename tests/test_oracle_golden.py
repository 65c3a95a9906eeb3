"""Pins the oracle's forward pass to the reference's golden fixture: NumPy
HF-Llama logits for a 2-layer bf16 checkpoint, 40 positions, tolerance 5e-4 and
zero argmax mismatches (tests/golden_parity_tests.rs:125-259)."""
import numpy as np

from helpers import compare_logits, load_golden, oracle_model

BLOCK = 16


def kv_for(cfg, blocks):
    return np.zeros(cfg.num_hidden_layers * blocks * BLOCK * cfg.num_key_value_heads * 2 * cfg.head_dim, np.float32)


def test_incremental_decode_matches_golden(oracle):
    cfg, tokens, golden, hw = load_golden()
    m = oracle_model(oracle, cfg, hw)
    nblocks = (len(tokens) + BLOCK - 1) // BLOCK
    # scattered, reversed physical blocks as the reference test allocates them
    table = list(range(nblocks + 2))[::-1][:nblocks]
    kv = kv_for(cfg, nblocks + 2)
    got = np.stack([m.forward(int(t), i, table, kv, BLOCK) for i, t in enumerate(tokens)])
    max_abs, mism = compare_logits(got, golden, oracle.argmax)
    assert max_abs < 5e-4 and mism == 0, (max_abs, mism)


def test_prefill_and_batched_prefill_match_golden_last_position(oracle):
    cfg, tokens, golden, hw = load_golden()
    m = oracle_model(oracle, cfg, hw)
    table = [2, 0, 1]
    want = None
    for chunk in (None, 1, 4, 16, 64):
        kv = kv_for(cfg, 3)
        if chunk is None:
            got = m.prefill(tokens, 0, table, kv, BLOCK)
            want = got
        else:
            got = m.prefill_batched(tokens, 0, table, kv, BLOCK, chunk)
            # batched == sequential bit for bit on the CPU path (README:359-364)
            assert np.array_equal(got, want), chunk
        assert np.abs(got - golden[-1]).max() < 5e-4
        assert oracle.argmax(got) == oracle.argmax(golden[-1])


def test_split_prefill_equals_whole(oracle):  # golden_parity_tests.rs:217-259
    cfg, tokens, golden, hw = load_golden()
    m = oracle_model(oracle, cfg, hw)
    table = [0, 1, 2]
    kv_a, kv_b = kv_for(cfg, 3), kv_for(cfg, 3)
    whole = m.prefill(tokens, 0, table, kv_a, BLOCK)
    m.prefill(tokens[:23], 0, table, kv_b, BLOCK)
    split = m.prefill(tokens[23:], 23, table, kv_b, BLOCK)
    assert np.abs(whole - split).max() < 1e-5


def test_batched_decode_equals_single_sequence(oracle):  # batched_decode_tests.rs:158-263
    cfg, tokens, golden, hw = load_golden()
    for quant in ("f32", "int8"):
        m = oracle_model(oracle, cfg, hw, quant)
        lens = [5, 17, 16, 30]
        kv_b, kv_s = kv_for(cfg, 12), kv_for(cfg, 12)
        tables = [[3 * b + i for i in range(3)] for b in range(4)]
        for b, n in enumerate(lens):
            m.prefill(tokens[:n], 0, tables[b], kv_b, BLOCK)
            m.prefill(tokens[:n], 0, tables[b], kv_s, BLOCK)
        nxt = [int(tokens[n]) for n in lens]
        got = m.decode_batch(nxt, lens, tables, kv_b, BLOCK)
        for b, n in enumerate(lens):
            solo = m.forward(nxt[b], n, tables[b], kv_s, BLOCK)
            assert np.array_equal(got[b], solo), (quant, b)
        assert np.array_equal(kv_b, kv_s)


def test_int8_model_is_smaller_and_tracks_f32(oracle):  # engine_tests.rs:331-375
    cfg, tokens, golden, hw = load_golden()
    f = oracle_model(oracle, cfg, hw, "f32")
    q = oracle_model(oracle, cfg, hw, "int8", lm_head_int8=True)
    assert f.weight_bytes() >= 3 * q.weight_bytes()
    kv = kv_for(cfg, 3)
    got = np.stack([q.forward(int(t), i, [0, 1, 2], kv, BLOCK) for i, t in enumerate(tokens)])
    agree = sum(int(oracle.argmax(a) == oracle.argmax(e)) for a, e in zip(got, golden))
    assert agree >= len(tokens) // 2
    assert np.abs(got - golden).max() < 0.25
