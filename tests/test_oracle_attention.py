"""The oracle's grouped-lane paged attention against a naive per-head reference,
restating tests/attention_tests.rs (bit-identical across lane widths; windows;
unmapped blocks; shared tables; zero-width window; oversize score stride)."""
import numpy as np

from helpers import AttnCase


def lane_widths(g):
    return [d for d in range(1, g + 1) if g % d == 0]


def run(oracle, case, q, tables, positions, starts, d, stride=None):
    L = oracle.kv_layout(1, case.total_blocks, case.block_size, case.num_kv_heads, case.head_dim)
    return oracle.paged_attention(q, case.kv_cache, L, case.num_heads, tables, positions, starts,
                                  heads_per_lane=d, score_stride=stride)


def test_every_lane_width_is_bit_identical_and_matches_naive(oracle):  # attention_tests.rs:168-194
    for H, KH in [(8, 1), (8, 2), (8, 4), (8, 8), (6, 3), (12, 4)]:
        for batch in (1, 3):
            case = AttnCase(H, KH, 4, 8, batch, 5, 5)
            pos = [39 - b * 9 for b in range(batch)]
            st = case.starts(pos, None)
            outs = [run(oracle, case, case.q, case.tables, pos, st, d) for d in lane_widths(H // KH)]
            for o in outs[1:]:
                assert np.array_equal(o, outs[0])
            naive = case.naive(case.q, case.tables, pos, st)
            assert np.allclose(outs[0], naive, rtol=1e-5, atol=1e-6)


def test_windows_and_block_boundaries(oracle):  # attention_tests.rs:197-225
    case = AttnCase(8, 2, 4, 8, 1, 6, 6)
    for pos in range(0, 48, 5):
        for window in (None, 1, 2, 7, 8, 9, 16, 33):
            st = case.starts([pos], window)
            outs = [run(oracle, case, case.q, case.tables, [pos], st, d) for d in lane_widths(4)]
            for o in outs[1:]:
                assert np.array_equal(o, outs[0])
            assert np.allclose(outs[0], case.naive(case.q, case.tables, [pos], st), rtol=1e-5, atol=1e-6)


def test_unmapped_positions_are_masked(oracle):  # attention_tests.rs:228-253
    case = AttnCase(8, 2, 4, 8, 1, 6, 2)
    full = run(oracle, case, case.q, case.tables, [40], [0], 4)
    trunc = run(oracle, case, case.q, case.tables, [15], [0], 4, stride=16)
    assert np.array_equal(full, trunc)
    assert np.all(np.isfinite(full))


def test_shared_table_entries_stay_independent(oracle):  # attention_tests.rs:279-322
    case = AttnCase(8, 2, 4, 8, 3, 5, 5)
    positions = [7, 19, 33]
    shared = [case.tables[0]] * 3
    got = run(oracle, case, case.q, shared, positions, [0, 0, 0], 4)
    per = 8 * 4
    for i, p in enumerate(positions):
        solo = run(oracle, case, case.q[i * per:(i + 1) * per], [case.tables[0]], [p], [0], 2)
        assert np.array_equal(got[i], solo[0])


def test_zero_width_window_gives_zeros(oracle):  # attention_tests.rs:325-341
    case = AttnCase(8, 2, 4, 8, 1, 4, 4)
    out = run(oracle, case, case.q, case.tables, [20], [21], 2, stride=1)
    assert np.all(out == 0.0)


def test_oversize_score_stride_is_harmless(oracle):  # attention_tests.rs:344-363
    case = AttnCase(8, 2, 4, 8, 2, 5, 5)
    pos = [9, 34]
    tight = 35
    want = run(oracle, case, case.q, case.tables, pos, [0, 0], 4, stride=tight)
    for stride in (tight + 1, tight + 17, tight * 2):
        for d in lane_widths(4):
            assert np.array_equal(run(oracle, case, case.q, case.tables, pos, [0, 0], d, stride=stride), want)


def test_lane_width_rule(oracle):  # attention.rs:381-408
    L = oracle.lib()
    for threads in (1, 4, 8):
        want = threads * 2
        for g in (1, 2, 4, 5, 8, 16):
            for kvh in (1, 2, 4, 8):
                for batch in (1, 2, 8, 32):
                    d = L.orc_lane_width(g, kvh, batch, threads, 2)
                    assert d >= 1 and g % d == 0
                    assert batch * kvh * (g // d) >= want or d == 1
                    for wider in range(d + 1, g + 1):
                        if g % wider == 0:
                            assert batch * kvh * (g // wider) < want
