"""Known-answer vectors of tests/math_tests.rs against the oracle, plus the
quantiser's edge cases (src/math.rs:456-469)."""
import numpy as np

from helpers import seq


def test_rms_norm_known_answer(oracle):  # math_tests.rs:36-49
    got = oracle.rms_norm([1.0, 2.0, 3.0, 4.0], [0.5] * 4, 1e-5)
    assert np.allclose(got, [0.182574, 0.365148, 0.547722, 0.730296], atol=1e-5)


def test_silu_and_swiglu_known_answers(oracle):  # math_tests.rs:52-72
    assert abs(oracle.silu(2.0) - 1.761594) < 1e-5
    got = oracle.swiglu([1.0, -1.0, 2.0], [2.0, 0.5, -1.0])
    assert np.allclose(got, [1.462117, -0.134470, -1.761594], atol=1e-5)


def test_rope_interleaved_known_answer(oracle):  # math_tests.rs:75-103
    got = oracle.apply_rope([1.0, 0.0, 1.0, 0.0], 1, 10000.0, style=1)
    assert np.allclose(got, [0.540302, 0.841470, 0.999950, 0.0099998], atol=1e-5)


def test_rope_neox_known_answer(oracle):  # math_tests.rs:105-122
    got = oracle.apply_rope([1.0, 1.0, 0.0, 0.0], 1, 10000.0, style=0)
    assert np.allclose(got, [0.540302, 0.999950, 0.841470, 0.0099998], atol=1e-5)


def test_rope_conventions_differ_and_preserve_norm(oracle):  # math_tests.rs:125-162
    base = (np.arange(8, dtype=np.float32) + 1) * np.float32(0.3)
    a = oracle.apply_rope(base, 5, 10000.0, 0)
    b = oracle.apply_rope(base, 5, 10000.0, 1)
    assert np.abs(a - b).max() > 0.1
    for style in (0, 1):
        v = np.array([((i * 7 % 5) - 2.0) for i in range(16)], np.float32)
        r = oracle.apply_rope(v, 13, 10000.0, style)
        assert abs(float((v * v).sum()) - float((r * r).sum())) < 1e-4


def test_softmax_masks(oracle):  # math_tests.rs:165-181, :190-196
    assert np.all(oracle.softmax([-np.inf] * 4) == 0.0)
    s = oracle.softmax([1.0, -np.inf, 1.0])
    assert s[1] == 0.0 and abs(s[0] - 0.5) < 1e-6 and abs(s[2] - 0.5) < 1e-6
    s = oracle.softmax([1.0, 2.0, 3.0])
    assert abs(s.sum() - 1.0) < 1e-6 and s[2] > s[1] > s[0]


def test_axpy_accumulates(oracle):  # math_tests.rs:183-188
    out = np.array([1.0, 2.0, 3.0], np.float32)
    oracle.axpy(out, 2.0, [0.5, -1.0, 4.0])
    assert np.allclose(out, [2.0, 0.0, 11.0], atol=1e-6)


def test_quantize_roundtrip(oracle):  # math_tests.rs:237-264
    rows, cols = 4, 8
    w = ((np.arange(rows * cols, dtype=np.float32) / np.float32(rows * cols)) * 2 - 1).astype(np.float32)
    q, s = oracle.quantize_rows_i8(w, rows, cols)
    deq = q.astype(np.float32) * s[:, None]
    assert np.abs(deq - w.reshape(rows, cols)).max() < max(0.01 * np.abs(w).max(), 1e-4)


def test_quantize_edges(oracle):
    w = np.zeros((5, 8), np.float32)
    w[1] = [0.5, -0.5, 0.25, 0, 0, 0, 0, 1e-9]          # +-absmax -> +-127
    w[2] = [3.0, 0.0118110236, -0.0118110236, 1.5, -1.5, 2.9999, 1e-30, -3.0]  # near-half codes
    w[3, 0] = np.float32(1e-38)                           # subnormal-scale row
    w[4] = [np.inf, 1.0, -1.0, 0, 0, 0, 0, -np.inf]       # inf absmax: finite entries -> 0, inf -> nan -> 0
    q, s = oracle.quantize_rows_i8(w, 5, 8)
    assert s[0] == 1.0 and np.all(q[0] == 0)              # all-zero row keeps scale 1.0
    assert q[1, 0] == 127 and q[1, 1] == -127 and s[1] == np.float32(0.5) / np.float32(127)
    # numpy restatement: true division, round half away from zero, clamp.
    for r in (1, 2, 3):
        sc = s[r]
        v = w[r] / sc
        want = np.clip(np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)), -127, 127).astype(np.int8)
        assert np.array_equal(q[r], want), r
    assert np.all(np.abs(q.astype(np.int32)) <= 127)


def test_matvec_i8_matches_f32_within_two_percent(oracle):  # math_tests.rs:267-295
    rows, cols = 16, 32
    x = (np.arange(cols, dtype=np.float32) * np.float32(0.01) - np.float32(0.15)).astype(np.float32)
    w = ((np.arange(rows * cols) % 37).astype(np.float32) * np.float32(0.01) - np.float32(0.18)).reshape(rows, cols)
    q, s = oracle.quantize_rows_i8(w, rows, cols)
    f = oracle.matvec_f32(x, w)
    i8 = oracle.matvec_i8(x, q, s)
    rel = np.where(np.abs(f) > 1e-6, np.abs(f - i8) / np.abs(f), np.abs(f - i8))
    assert rel.max() < 0.02


def test_argmax_breaks_ties_toward_the_last_index(oracle):  # sampling.rs:140-147
    assert oracle.argmax([1.0, 3.0, 3.0, 2.0]) == 2
    assert oracle.argmax([5.0]) == 0
    assert oracle.argmax([0.0, -0.0]) == 0          # total_cmp: -0.0 < +0.0
    assert oracle.argmax([-0.0, 0.0]) == 1
    assert oracle.argmax([1.0, np.nan, 2.0]) == 1   # positive NaN sorts above everything


def test_kv_layout_is_dense_and_copy_block_copies_all_layers(oracle):  # layout.rs:99-177
    L = oracle.kv_layout(3, 4, 2, 2, 4)
    seen = set()
    for layer in range(3):
        for blk in range(4):
            for tok in range(2):
                for h in range(2):
                    for v in (0, 1):
                        seen.add(oracle.kv_index(L, layer, blk, tok, h, v))
    assert len(seen) == L.total_floats() // 4 and max(seen) == L.total_floats() - 4
    cache = np.arange(L.total_floats(), dtype=np.float32)
    before = cache.copy()
    oracle.kv_copy_block(L, cache, 1, 3)
    c = cache.reshape(3, 4, -1)
    assert np.array_equal(c[:, 3], before.reshape(3, 4, -1)[:, 1])
    assert np.array_equal(c[:, :3], before.reshape(3, 4, -1)[:, :3])
    import pytest
    with pytest.raises(ValueError):
        oracle.kv_copy_block(L, cache, 2, 2)
