"""The tcgen05 tensor-core dequant GEMM (batches beyond a few rows) against the
oracle's int8 CPU matmat and against the library's own CUDA-core path.

Tolerance: 2e-5 relative to max(|expected|, 1), scaled by sqrt(K/2048): the
activations enter the tensor cores as three bf16 planes whose sum is the f32
value exactly and accumulate in f32, so only the summation order differs from
the CPU kernel."""
import numpy as np
import pytest

from helpers import normal_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from paged_infer_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def rel_err(got, want):
    return float((np.abs(got - want) / np.maximum(np.abs(want), 1.0)).max())


@pytest.mark.parametrize("rows,cols", [(2048, 2048), (256, 2048), (2560, 2048), (2048, 5632), (1000, 256), (32000, 2048)])
@pytest.mark.parametrize("M", [5, 16, 17, 64, 130])
def test_tensor_gemm_matches_cpu_matmat(ctx, oracle, rows, cols, M):
    from paged_infer_b200 import api
    w = normal_f32((rows, cols), rows + cols, 0.02)
    q, s = oracle.quantize_rows_i8(w, rows, cols)
    x = normal_f32((M, cols), M, 1.0)
    x[0] *= 1e-6          # rows of very different magnitude: the planes carry any exponent
    x[-1] *= 3e4
    x[1, ::7] = 0.0
    p = api.Projection.int8(ctx, q, s)
    want = oracle.matmat_i8(x, q, s)
    got = p.apply_batched(x)
    tol = 2e-5 * max(1.0, (cols / 2048.0) ** 0.5)
    scale = np.maximum(np.abs(x).max(axis=1, keepdims=True), 1e-30)   # compare per activation row, relative to its size
    assert rel_err(got / scale, want / scale) < tol
    # and the CUDA-core path agrees with it
    ctx.set_option(api._lib.PI_OPT_TENSOR_GEMM, 0)
    try:
        slow = p.apply_batched(x)
    finally:
        ctx.set_option(api._lib.PI_OPT_TENSOR_GEMM, 1)
    assert rel_err(got / scale, slow / scale) < tol


def test_extreme_magnitudes_stay_f32_equivalent(ctx, oracle):
    """Activations travel as three bf16 planes whose sum is the f32 value exactly: huge, tiny and mixed rows
    (beyond the fp16 range in both directions) give the same relative accuracy as ordinary ones."""
    from paged_infer_b200 import api
    rows, cols, M = 2048, 2048, 24
    q, s = oracle.quantize_rows_i8(normal_f32((rows, cols), 77, 0.02), rows, cols)
    x = normal_f32((M, cols), 78, 1.0)
    x[0] *= 1e30
    x[1] *= 1e-30
    x[2, ::2] *= 1e12       # 24 binades between neighbours
    x[3, ::3] *= 1e-12
    x[4] = 0.0
    p = api.Projection.int8(ctx, q, s)
    want = oracle.matmat_i8(x, q, s)
    got = p.apply_batched(x)
    scale = np.maximum(np.abs(want).max(axis=1, keepdims=True), 1e-37)
    assert float(np.abs(got / scale - want / scale).max()) < 2e-5
    assert np.all(got[4] == 0.0)


def test_tensor_gemm_really_ran(ctx, oracle):
    from paged_infer_b200 import api
    q, s = oracle.quantize_rows_i8(normal_f32((512, 512), 1, 0.02), 512, 512)
    p = api.Projection.int8(ctx, q, s)
    x = normal_f32((32, 512), 2, 1.0)
    ctx.profile_begin()
    p.apply_batched(x)
    prof = ctx.profile_end()
    assert prof["gemm_tc"][1] == 1 and prof["gemv"][1] == 0
    ctx.profile_begin()
    p.apply_batched(x[:2])
    prof = ctx.profile_end()
    assert prof["gemm_tc"][1] == 0 and prof["gemv"][1] == 1


def test_results_do_not_depend_on_timing(ctx, oracle):
    """Split-K partial sums are added in a fixed order: repeated launches are bit-identical."""
    from paged_infer_b200 import api
    q, s = oracle.quantize_rows_i8(normal_f32((2048, 5632), 3, 0.02), 2048, 5632)
    p = api.Projection.int8(ctx, q, s)
    x = normal_f32((64, 5632), 4, 1.0)
    first = p.apply_batched(x)
    for _ in range(5):
        assert np.array_equal(p.apply_batched(x), first)
