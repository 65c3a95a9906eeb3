"""The oracle's vector kernels against its scalar ones, restating
tests/simd_tests.rs: every length across the unroll boundaries, the int8 range
edges, and the bit-identity of the tiled kernels with the single dot."""
import numpy as np
import pytest

from helpers import seq, seq_i8


def close(a, e):
    return abs(a - e) / max(abs(e), 1.0) < 1e-5


def test_reports_a_backend(oracle):
    assert oracle.backend() in ("avx2+fma", "scalar")


def test_dot_and_dot_i8_match_scalar_at_every_length(oracle):  # simd_tests.rs:53-78
    for n in range(80):
        a, b = seq(n, 1), seq(n, 7)
        assert close(oracle.dot(a, b), oracle.dot_scalar(a, b)), n
        w, x = seq_i8(n, 3), seq(n, 11)
        assert close(oracle.dot_i8(w, x), oracle.dot_i8_scalar(w, x)), n


def test_scalar_kernels_follow_the_four_accumulator_order(oracle):
    # dot_i8_scalar (simd.rs:60-77) restated in numpy f32, element by element.
    for n in (0, 1, 5, 8, 33, 79):
        w, x = seq_i8(n, 3), seq(n, 11)
        acc = np.zeros(4, np.float32)
        i = 0
        while i + 4 <= n:
            for j in range(4):
                acc[j] = np.float32(acc[j] + np.float32(np.float32(w[i + j]) * x[i + j]))
            i += 4
        total = np.float32(np.float32(acc[0] + acc[1]) + np.float32(acc[2] + acc[3]))
        while i < n:
            total = np.float32(total + np.float32(np.float32(w[i]) * x[i]))
            i += 1
        assert oracle.dot_i8_scalar(w, x) == total


def test_axpy_matches_scalar(oracle):  # simd_tests.rs:80-94
    for n in range(80):
        v, base = seq(n, 5), seq(n, 13)
        got = base.copy()
        oracle.axpy(got, 0.375, v)
        want = base + np.float32(0.375) * v
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6)


def test_extreme_magnitudes(oracle):  # simd_tests.rs:96-103
    a = np.array([1e-8, 1e8, -1e-8, -1e8, 3.0, 0.0, -7.5, 2.25, 1.0], np.float32)
    b = np.array([1e8, 1e-8, 1e8, 1e-8, 2.0, 5.0, 4.0, -1.0, 6.0], np.float32)
    assert close(oracle.dot(a, b), oracle.dot_scalar(a, b))


def test_i8_sign_extension(oracle):  # simd_tests.rs:105-111
    w = np.array([-128, 127, -1, 0, 1, -128, 127, -1, 5], np.int8)
    assert close(oracle.dot_i8(w, np.ones(9, np.float32)), float(w.astype(np.float32).sum()))


def test_dot_multi_is_dot_bit_for_bit(oracle):  # simd_tests.rs:186-220
    def mk(seed, n):
        i = np.arange(n)
        return (((i * 37 + seed * 101) % 251).astype(np.float32) * np.float32(0.013) - np.float32(1.6)).astype(np.float32)

    for n in [0, 1, 3, 4, 7, 8, 9, 15, 16, 17, 31, 32, 33, 40, 63, 64, 65, 96, 129]:
        w = mk(0, n)
        for bt in range(1, 7):
            block = np.concatenate([mk(b + 1, n) for b in range(bt)]) if n else np.zeros(0, np.float32)
            expect = np.array([oracle.dot(w, block[b * n:(b + 1) * n]) for b in range(bt)], np.float32)
            got = oracle.dot_multi(w, block, n, bt)
            assert np.array_equal(got, expect), (n, bt)


def test_dot_i8_multi_is_dot_i8_bit_for_bit(oracle):  # simd_tests.rs:241-272
    for n in [0, 1, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 40, 64, 65, 96, 129]:
        w = np.array([(-128 if i % 5 == 0 else 127 if i % 5 == 1 else -1 if i % 5 == 2 else 0 if i % 5 == 3
                       else ((i * 31) % 127)) for i in range(n)], np.int8)
        for bt in (1, 2, 3, 4):
            i = np.arange(bt * n)
            block = (((i * 17) % 211).astype(np.float32) * np.float32(0.011) - np.float32(1.2)).astype(np.float32)
            expect = np.array([oracle.dot_i8(w, block[b * n:(b + 1) * n]) for b in range(bt)], np.float32)
            got = oracle.dot_i8_multi(w, block, n, bt)
            assert np.array_equal(got, expect), (n, bt)


def test_parallel_matvec_matches_sequential(oracle):  # simd_tests.rs:113-129
    for rows, cols in [(1, 1), (3, 7), (8, 32), (17, 33), (64, 129), (129, 64)]:
        w = seq(rows * cols, 21).reshape(rows, cols)
        x = seq(cols, 42)
        fast = oracle.matvec_f32(x, w)
        ref = oracle.matvec_f32(x, w, sequential=True)
        assert all(close(f, s) for f, s in zip(fast, ref))


def test_int8_matvec_tracks_f32(oracle):  # simd_tests.rs:131-150
    rows, cols = 48, 96
    w = seq(rows * cols, 77).reshape(rows, cols)
    x = seq(cols, 99)
    q, s = oracle.quantize_rows_i8(w, rows, cols)
    f = oracle.matvec_f32(x, w)
    i8 = oracle.matvec_i8(x, q, s)
    assert np.all(np.abs(f - i8) / np.maximum(np.abs(f), 1e-3) < 0.02)


def test_matmat_equals_matvec_per_entry_bit_for_bit(oracle):
    # The batched kernel is a scheduling change only (README "bit-identical";
    # math.rs:223-275 over dot_i8_multi<4|2> and dot_i8).
    rows, cols = 37, 136
    w = seq(rows * cols, 5).reshape(rows, cols)
    q, s = oracle.quantize_rows_i8(w, rows, cols)
    for batch in (1, 2, 3, 4, 5, 7, 8, 11):
        x = seq(batch * cols, 9 + batch).reshape(batch, cols)
        got = oracle.matmat_i8(x, q, s)
        want = np.stack([oracle.matvec_i8(x[b], q, s) for b in range(batch)])
        assert np.array_equal(got, want), batch
        gotf = oracle.matmat_f32(x, w)
        wantf = np.stack([oracle.matvec_f32(x[b], w) for b in range(batch)])
        assert np.array_equal(gotf, wantf), batch
        assert np.array_equal(oracle.matmat_i8(x, q, s, tile=1), want)
