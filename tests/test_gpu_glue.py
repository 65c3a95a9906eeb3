"""Per-token glue on the GPU: the known answers of tests/math_tests.rs and
parity with the oracle (1e-6 absolute + 1e-6 relative: these are elementwise
f32 ops whose only differences are libm ulps and reduction order)."""
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


def test_rms_norm(ctx, oracle):
    from paged_infer_b200 import api
    got = api.rms_norm(ctx, [1.0, 2.0, 3.0, 4.0], [0.5] * 4, 1e-5)
    assert np.allclose(got, [0.182574, 0.365148, 0.547722, 0.730296], atol=1e-5)
    for n in (1, 24, 96, 2048, 5000):
        x = normal_f32((5, n), n, 1.0)
        w = 1 + normal_f32(n, n + 1, 0.1)
        got = api.rms_norm(ctx, x, w, 1e-5)
        want = np.stack([oracle.rms_norm(r, w, 1e-5) for r in x])
        assert np.allclose(got, want, rtol=2e-6, atol=1e-6), n
    with pytest.raises(api.PiError):
        api.rms_norm(ctx, np.ones(4), np.ones(3), 1e-5)


def test_swiglu(ctx, oracle):
    from paged_infer_b200 import api
    got = api.swiglu(ctx, [1.0, -1.0, 2.0], [2.0, 0.5, -1.0])
    assert np.allclose(got, [1.462117, -0.134470, -1.761594], atol=1e-5)
    g, u = normal_f32(5632 * 3, 1, 2.0), normal_f32(5632 * 3, 2, 1.0)
    assert np.allclose(api.swiglu(ctx, g, u), oracle.swiglu(g, u), rtol=2e-6, atol=1e-7)
    with pytest.raises(api.PiError):
        api.swiglu(ctx, np.ones(4), np.ones(3))


def test_rope_known_answers_and_styles(ctx, oracle):
    from paged_infer_b200 import api
    got = api.apply_rope(ctx, [1.0, 0.0, 1.0, 0.0], 1, 4, 10000.0, style=1)
    assert np.allclose(got, [0.540302, 0.841470, 0.999950, 0.0099998], atol=1e-5)
    got = api.apply_rope(ctx, [1.0, 1.0, 0.0, 0.0], 1, 4, 10000.0, style=0)
    assert np.allclose(got, [0.540302, 0.999950, 0.841470, 0.0099998], atol=1e-5)
    base = (np.arange(8, dtype=np.float32) + 1) * np.float32(0.3)
    a = api.apply_rope(ctx, base, 5, 8, 10000.0, 0)
    b = api.apply_rope(ctx, base, 5, 8, 10000.0, 1)
    assert np.abs(a - b).max() > 0.1
    for style in (0, 1):
        for hd, theta in ((64, 10000.0), (128, 500000.0), (24, 10000.0)):
            x = normal_f32((6, 3 * hd), hd + style, 1.0)
            pos = np.array([0, 1, 17, 255, 2047, 4095], np.int32)
            got = api.apply_rope(ctx, x, pos, hd, theta, style)
            want = np.stack([np.concatenate([oracle.apply_rope(r[h * hd:(h + 1) * hd], int(p), theta, style)
                                             for h in range(3)]) for r, p in zip(x, pos)])
            # the angles come from the same host libm; only the rotation's mul/add rounding can differ
            assert np.allclose(got, want, rtol=0, atol=1e-6), (style, hd)
            assert np.allclose((got * got).sum(1), (x * x).sum(1), rtol=1e-5)


def test_argmax_ties_go_to_the_last_index(ctx, oracle):
    from paged_infer_b200 import api
    assert api.argmax(ctx, [1.0, 3.0, 3.0, 2.0]) == 2
    assert api.argmax(ctx, [5.0]) == 0
    assert api.argmax(ctx, [0.0, -0.0]) == 0 and api.argmax(ctx, [-0.0, 0.0]) == 1
    l = normal_f32((7, 32000), 3, 0.9)
    l[2, [5, 31999]] = 50.0
    l[3, [0, 1, 2]] = 60.0
    l[4, :] = -1.5
    got = api.argmax(ctx, l)
    assert got.tolist() == [oracle.argmax(r) for r in l]
    assert got[2] == 31999 and got[3] == 2 and got[4] == 31999
