"""Quantiser and projections on the GPU against the oracle (through the C ABI).

Bars: int8 codes and scales bit-exact (reference src/math.rs:456-469);
projection outputs within 1e-5 relative to max(|expected|, 1) of the oracle's
int8/f32 CPU matvec / matmat (the tolerance tests/simd_tests.rs:36-42 uses for
re-associated sums), scaled by sqrt(K/2048) for long rows."""
import numpy as np
import pytest

from helpers import normal_f32, seq

pytestmark = pytest.mark.gpu

TL_SHAPES = [(2048, 2048), (256, 2048), (5632, 2048), (2048, 5632), (32000, 2048)]


@pytest.fixture(scope="module")
def ctx():
    from paged_infer_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def assert_close(got, want, K, what=""):
    tol = 1e-5 * max(1.0, (K / 2048.0) ** 0.5) * 4
    err = np.abs(got - want) / np.maximum(np.abs(want), 1.0)
    assert err.max() < tol, f"{what}: max rel err {err.max():.3e} > {tol:.1e}"


@pytest.mark.parametrize("rows,cols", TL_SHAPES + [(48, 96), (112, 96), (96, 192), (17, 33), (64, 129), (1, 1), (3, 7)])
def test_quantize_is_bit_exact(ctx, oracle, rows, cols):
    from paged_infer_b200 import api
    w = normal_f32((rows, cols), 1000 + rows + cols, 0.02)
    if rows > 4:
        w[1] = 0.0                      # all-zero row keeps scale 1.0
        w[2, 0] = np.abs(w[2]).max() * 2  # +absmax -> +127 exactly
        w[3, -1] = -np.abs(w[3]).max() * 3
    q, s = api.quantize_rows_i8(ctx, w, rows, cols)
    qo, so = oracle.quantize_rows_i8(w, rows, cols)
    assert np.array_equal(s.view(np.uint32), so.view(np.uint32))
    assert np.array_equal(q, qo)
    if rows > 4:
        assert s[1] == 1.0 and not q[1].any() and q[2, 0] == 127 and q[3, -1] == -127


def test_quantize_special_values(ctx, oracle):
    from paged_infer_b200 import api
    w = np.zeros((6, 16), np.float32)
    w[0, :4] = [np.inf, 1.0, -1.0, -np.inf]
    w[1, :4] = [np.nan, 2.0, -1.0, 0.5]
    w[2, :3] = [1e-38, -1e-39, 5e-39]
    w[3, :5] = [127.0, 0.5, 1.5, -0.5, -2.5]       # scale 1.0: exact halves round away from zero
    w[4] = np.linspace(-3e38, 3e38, 16, dtype=np.float32)
    w[5, :2] = [-0.0, 1e-45]
    q, s = api.quantize_rows_i8(ctx, w, 6, 16)
    qo, so = oracle.quantize_rows_i8(w, 6, 16)
    assert np.array_equal(s.view(np.uint32), so.view(np.uint32))
    assert np.array_equal(q, qo)
    assert q[3, :5].tolist() == [127, 1, 2, -1, -3]


def test_from_packed_matches_host_quantiser_and_reads_back(ctx, oracle):
    from paged_infer_b200 import api
    w = normal_f32((300, 130), 7, 0.02)
    p = api.Projection.from_packed(ctx, w)
    q, s = p.read_i8()
    qo, so = oracle.quantize_rows_i8(w, 300, 130)
    assert np.array_equal(q, qo) and np.array_equal(s, so)
    assert p.rows() == 300 and p.cols() == 130 and p.weight_bytes() == 300 * 130 + 4 * 300 and p.is_int8()


@pytest.mark.parametrize("rows,cols", TL_SHAPES)
def test_int8_matvec_tinyllama_shapes(ctx, oracle, rows, cols):
    from paged_infer_b200 import api
    w = normal_f32((rows, cols), 1, 0.02)
    x = normal_f32(cols, 2, 1.0)
    q, s = oracle.quantize_rows_i8(w, rows, cols)
    p = api.Projection.int8(ctx, q, s)
    assert_close(p.apply_parallel(x), oracle.matvec_i8(x, q, s), cols, f"{rows}x{cols}")


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 9, 32])
def test_int8_batched_matches_matmat(ctx, oracle, M):
    from paged_infer_b200 import api
    for rows, cols in [(2048, 2048), (256, 2048), (2048, 5632)]:
        w = normal_f32((rows, cols), 3, 0.02)
        x = normal_f32((M, cols), 4 + M, 1.0)
        q, s = oracle.quantize_rows_i8(w, rows, cols)
        p = api.Projection.int8(ctx, q, s)
        assert_close(p.apply_batched(x), oracle.matmat_i8(x, q, s), cols, f"{rows}x{cols} M={M}")


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (8, 32), (17, 33), (64, 129), (129, 64), (48, 96), (112, 96), (96, 192), (33, 40)])
def test_odd_shapes_every_weight_kind(ctx, oracle, rows, cols):
    from paged_infer_b200 import api
    from paged_infer_b200.loader import bf16_bits_to_f32, f32_to_bf16_bits
    w = seq(rows * cols, 21).reshape(rows, cols)
    for M in (1, 3, 6):
        x = seq(M * cols, 42 + M).reshape(M, cols)
        # f32 weights: Projection::F32
        assert_close(api.Projection.f32(ctx, w).apply_batched(x), oracle.matmat_f32(x, w), cols, "f32")
        # bf16 checkpoint weights widened exactly
        bits = f32_to_bf16_bits(w)
        assert_close(api.Projection.f32(ctx, bits).apply_batched(x), oracle.matmat_f32(x, bf16_bits_to_f32(bits)), cols, "bf16")
        # int8
        q, s = oracle.quantize_rows_i8(w, rows, cols)
        assert_close(api.Projection.int8(ctx, q, s).apply_batched(x), oracle.matmat_i8(x, q, s), cols, "int8")


def test_i8_range_edges_and_row_independence(ctx, oracle):
    from paged_infer_b200 import api
    # i8::MIN must sign-extend to -128 (tests/simd_tests.rs:105-111)
    q = np.array([[-128, 127, -1, 0, 1, -128, 127, -1, 5]], np.int8)
    out = api.Projection.int8(ctx, q, np.ones(1, np.float32)).apply_parallel(np.ones(9, np.float32))
    assert out[0] == float(q.astype(np.float32).sum())
    # zeroing one weight row changes exactly that output (tests/simd_tests.rs:153-184)
    rows, cols = 33, 40
    w = seq(rows * cols, 5).reshape(rows, cols)
    x = seq(cols, 6)
    base = api.Projection.f32(ctx, w).apply_parallel(x)
    assert np.all(np.isfinite(base))
    w2 = w.copy()
    w2[10] = 0
    out2 = api.Projection.f32(ctx, w2).apply_parallel(x)
    assert out2[10] == 0.0
    assert np.array_equal(np.delete(out2, 10), np.delete(base, 10))


def test_int8_tracks_f32_within_two_percent(ctx, oracle):
    from paged_infer_b200 import api
    rows, cols = 48, 96  # tests/simd_tests.rs:131-150
    w = seq(rows * cols, 77).reshape(rows, cols)
    x = seq(cols, 99)
    f = api.Projection.f32(ctx, w).apply_parallel(x)
    i8 = api.Projection.from_packed(ctx, w).apply_parallel(x)
    assert np.all(np.abs(f - i8) / np.maximum(np.abs(f), 1e-3) < 0.02)


def test_shape_errors_are_reported_not_fatal(ctx):
    from paged_infer_b200 import api
    p = api.Projection.f32(ctx, np.ones((4, 8), np.float32))
    with pytest.raises(api.PiError):
        p.apply_parallel(np.ones(7, np.float32))
    with pytest.raises(api.PiError):
        api.Projection.int8(ctx, np.ones((4, 8), np.int8), np.ones(3, np.float32))
    # the context is still usable
    assert np.allclose(p.apply_parallel(np.ones(8, np.float32)), 8.0)
