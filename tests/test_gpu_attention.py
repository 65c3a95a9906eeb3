"""Paged attention on the GPU against the oracle's PagedAttention::run and the
naive per-head reference, restating tests/attention_tests.rs, plus the KV pool
calls.  Tolerance 1e-5 relative to max(|expected|, 1): the GPU keeps an online
softmax and a different summation order, the arithmetic is otherwise the same."""
import numpy as np
import pytest

from helpers import AttnCase, normal_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from paged_infer_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def gpu_run(ctx, case, q, tables, positions, starts, layer=0):
    from paged_infer_b200 import api
    L = api.KvLayout(case.num_layers, case.total_blocks, case.block_size, case.num_kv_heads, case.head_dim)
    kv = api.KvCache(ctx, L)
    kv.upload(case.kv_cache)
    entries = [api.AttnEntry(api.BlockTable(t), p, start=s) for t, p, s in zip(tables, positions, starts)]
    return api.PagedAttention(L, case.num_heads).run(q, kv, entries, layer)


def cpu_run(oracle, case, q, tables, positions, starts, layer=0):
    L = oracle.kv_layout(case.num_layers, case.total_blocks, case.block_size, case.num_kv_heads, case.head_dim)
    return oracle.paged_attention(q, case.kv_cache, L, case.num_heads, tables, positions, starts, layer=layer)


def close(got, want, tol=1e-5):
    err = np.abs(got - want) / np.maximum(np.abs(want), 1.0)
    assert err.max() < tol, err.max()


def test_reference_head_shapes_ragged_batches(ctx, oracle):  # attention_tests.rs:168-194
    for H, KH in [(8, 1), (8, 2), (8, 4), (8, 8), (6, 3), (12, 4)]:
        for batch in (1, 3):
            case = AttnCase(H, KH, 4, 8, batch, 5, 5)
            pos = [39 - b * 9 for b in range(batch)]
            st = [0] * batch
            got = gpu_run(ctx, case, case.q, case.tables, pos, st)
            close(got, cpu_run(oracle, case, case.q, case.tables, pos, st))
            close(got, case.naive(case.q, case.tables, pos, st))


def test_windows_and_block_boundaries(ctx, oracle):  # attention_tests.rs:197-225, :256-276
    case = AttnCase(8, 2, 4, 8, 1, 6, 6)
    for pos in range(0, 48, 3):
        for window in (None, 1, 2, 7, 8, 9, 16, 33):
            st = case.starts([pos], window)
            close(gpu_run(ctx, case, case.q, case.tables, [pos], st), cpu_run(oracle, case, case.q, case.tables, [pos], st))
    case = AttnCase(8, 4, 4, 16, 1, 4, 4)
    for pos in (0, 1, 15, 16, 17, 31, 47):
        for window in (1, 2, 3):
            st = case.starts([pos], window)
            close(gpu_run(ctx, case, case.q, case.tables, [pos], st), cpu_run(oracle, case, case.q, case.tables, [pos], st))


def test_unmapped_positions_are_masked_not_read(ctx, oracle):  # attention_tests.rs:228-253
    case = AttnCase(8, 2, 4, 8, 1, 6, 2)
    full = gpu_run(ctx, case, case.q, case.tables, [40], [0])
    trunc = gpu_run(ctx, case, case.q, case.tables, [15], [0])
    assert np.array_equal(full, trunc) and np.all(np.isfinite(full))
    close(full, cpu_run(oracle, case, case.q, case.tables, [40], [0]))
    # nothing mapped at all, and a window that lies wholly in the unmapped tail: zeros, not NaN
    assert np.all(gpu_run(ctx, case, case.q, [[]], [5], [0]) == 0.0)
    assert np.all(gpu_run(ctx, case, case.q, case.tables, [40], [30]) == 0.0)


def test_shared_table_entries_stay_independent(ctx, oracle):  # attention_tests.rs:279-322
    case = AttnCase(8, 2, 4, 8, 3, 5, 5)
    positions = [7, 19, 33]
    shared = [case.tables[0]] * 3
    got = gpu_run(ctx, case, case.q, shared, positions, [0, 0, 0])
    close(got, cpu_run(oracle, case, case.q, shared, positions, [0, 0, 0]))
    per = 8 * 4
    for i, p in enumerate(positions):
        solo = gpu_run(ctx, case, case.q[i * per:(i + 1) * per], [case.tables[0]], [p], [0])
        assert np.array_equal(got[i], solo[0])


def test_zero_width_window_is_zeros(ctx):  # attention_tests.rs:325-341
    case = AttnCase(8, 2, 4, 8, 1, 4, 4)
    assert np.all(gpu_run(ctx, case, case.q, case.tables, [20], [21]) == 0.0)


@pytest.mark.parametrize("hd,H,KH,bs", [(64, 32, 4, 16), (128, 32, 8, 16), (128, 8, 1, 16), (64, 4, 4, 16), (64, 8, 4, 8),
                                        (128, 4, 2, 32), (24, 4, 2, 16), (64, 12, 4, 16)])
def test_model_head_shapes_random_kv(ctx, oracle, hd, H, KH, bs):
    """TinyLlama / Llama-3 / Llama-2-70B head geometry (fast path) and the fixture's head_dim 24 (generic path)."""
    rng = np.random.default_rng(hd + H)
    batch, blocks_per_seq = 5, 9
    case = AttnCase(H, KH, hd, bs, batch, blocks_per_seq, blocks_per_seq, num_layers=2)
    case.kv_cache = normal_f32(case.kv_cache.size, 11, 1.0)
    q = normal_f32(batch * H * hd, 12, 1.0)
    pos = [int(p) for p in rng.integers(0, blocks_per_seq * bs, batch)]
    pos[0], pos[1] = 0, blocks_per_seq * bs - 1
    for window in (None, 3 * bs + 1):
        st = case.starts(pos, window)
        for layer in (0, 1):
            close(gpu_run(ctx, case, q, case.tables, pos, st, layer), cpu_run(oracle, case, q, case.tables, pos, st, layer))


def test_long_contexts_split_the_kv_axis(ctx, oracle):
    """Contexts long enough that one (sequence, kv head) is spread over several CTAs."""
    H, KH, hd, bs = 32, 4, 64, 16
    batch, blocks = 3, 160
    case = AttnCase(H, KH, hd, bs, batch, blocks, blocks)
    case.kv_cache = normal_f32(case.kv_cache.size, 5, 1.0)
    q = normal_f32(batch * H * hd, 6, 1.0)
    pos = [2559, 1030, 300]
    got = gpu_run(ctx, case, q, case.tables, pos, [0, 0, 0])
    close(got, cpu_run(oracle, case, q, case.tables, pos, [0, 0, 0]))
    got = gpu_run(ctx, case, q, case.tables, pos, [1500, 0, 299])
    close(got, cpu_run(oracle, case, q, case.tables, pos, [1500, 0, 299]))


@pytest.mark.parametrize("hd,H,KH,batch,blocks", [(64, 32, 4, 40, 100), (128, 32, 8, 12, 80), (128, 8, 1, 64, 100)])
def test_flat_work_list_ragged_batch(ctx, oracle, hd, H, KH, batch, blocks):
    """Batches with enough tiles go over the flat tile list (equal ranges per resident warp, partial results merged
    by the warp that finishes an entry last): ragged positions, windows, an empty window, an empty table, a table
    that ends before the position.  Same results as the oracle, the same bits run after run, and the per-entry grid
    (option off) agrees to rounding."""
    from paged_infer_b200 import _lib
    bs = 16
    rng = np.random.default_rng(hd * 7 + H)
    case = AttnCase(H, KH, hd, bs, batch, blocks, blocks)
    case.kv_cache = normal_f32(case.kv_cache.size, 21, 1.0)
    q = normal_f32(batch * H * hd, 22, 1.0)
    pos = [int(p) for p in rng.integers(bs * blocks // 4, bs * blocks, batch)]
    st = [0] * batch
    tables = [list(t) for t in case.tables]
    pos[0], pos[1], pos[2] = 0, bs * blocks - 1, bs * 7 + 15
    st[3] = pos[3] - 37                      # sliding window inside the context
    st[4] = pos[4] + 1                       # empty window
    tables[5] = []                           # nothing mapped
    tables[6] = tables[6][:pos[6] // bs // 2]   # the table ends long before the position
    st[7] = (pos[7] // bs) * bs              # window starts on the position's own block
    want = cpu_run(oracle, case, q, tables, pos, st)
    ctx.set_option(_lib.PI_OPT_ATTN_FLAT, 2)     # also for a single attention call (1: inside a model forward only)
    got = gpu_run(ctx, case, q, tables, pos, st)
    again = gpu_run(ctx, case, q, tables, pos, st)
    ctx.set_option(_lib.PI_OPT_ATTN_FLAT, 0)
    grid = gpu_run(ctx, case, q, tables, pos, st)
    ctx.set_option(_lib.PI_OPT_ATTN_FLAT, 1)
    close(got, want)
    close(grid, want)
    assert np.array_equal(got, again)
    assert np.all(got[4] == 0.0) and np.all(got[5] == 0.0)
    assert not np.array_equal(got, grid), "the flat work list was not used"


def test_kv_pool_roundtrip_copy_block_and_token_io(ctx, oracle):
    from paged_infer_b200 import api
    for (nl, nb, bs, kh, hd) in [(3, 5, 16, 4, 64), (2, 4, 8, 2, 24), (1, 3, 1, 1, 1)]:
        L = api.KvLayout(nl, nb, bs, kh, hd)
        host = normal_f32(L.total_floats(), 1, 1.0)
        kv = api.KvCache(ctx, L)
        kv.upload(host)
        assert np.array_equal(kv.download(), host)
        # copy-on-write copy across all layers == the reference's copy_block (layout.rs:82-96)
        want = host.copy()
        oracle.kv_copy_block(oracle.kv_layout(nl, nb, bs, kh, hd), want, 1, nb - 1)
        kv.copy_block(1, nb - 1)
        assert np.array_equal(kv.download(), want)
        with pytest.raises(api.PiError):
            kv.copy_block(2, 2)
        with pytest.raises(api.PiError):
            kv.copy_block(0, nb)
        k, v = normal_f32(kh * hd, 2), normal_f32(kh * hd, 3)
        kv.write_token(nl - 1, 0, bs - 1, k, v)
        rk, rv = kv.read_token(nl - 1, 0, bs - 1)
        assert np.array_equal(rk, k) and np.array_equal(rv, v)
        d = kv.download()
        for h in range(kh):
            i = L.index(nl - 1, 0, bs - 1, h, False)
            assert np.array_equal(d[i:i + hd], k[h * hd:(h + 1) * hd])
            j = L.index(nl - 1, 0, bs - 1, h, True)
            assert np.array_equal(d[j:j + hd], v[h * hd:(h + 1) * hd])


def test_bad_head_grouping_is_an_error(ctx):
    from paged_infer_b200 import api
    L = api.KvLayout(1, 4, 8, 3, 4)
    kv = api.KvCache(ctx, L)
    with pytest.raises(api.PiError):  # 8 heads over 3 kv heads (attention.rs:159-165)
        api.PagedAttention(L, 8).run(np.zeros(8 * 4, np.float32), kv, [api.AttnEntry(api.BlockTable([0]), 3)])
    with pytest.raises(api.PiError):  # physical block outside the pool
        api.PagedAttention(L, 6).run(np.zeros(6 * 4, np.float32), kv, [api.AttnEntry(api.BlockTable([9]), 3)])


# ---- entries that share one block table (prefill chunks, speculative verify groups) ---------------------------

def shared_table_case(ctx, oracle, hd, H, KH, positions, starts, mapped_blocks, seed, layers=1, layer=0):
    """All entries map the same table; returns (decode-kernel result, shared-table-kernel result, oracle result)."""
    from paged_infer_b200 import api
    n = len(positions)
    blocks = max(positions) // 16 + 2
    case = AttnCase(H, KH, hd, 16, 1, blocks, min(mapped_blocks, blocks), num_layers=layers)
    case.kv_cache = normal_f32(case.kv_cache.size, seed, 1.0)
    q = normal_f32(n * H * hd, seed + 1, 1.0)
    tables = [case.tables[0]] * n
    want = cpu_run(oracle, case, q, tables, positions, starts, layer)
    ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, 0)
    try:
        per_entry = gpu_run(ctx, case, q, tables, positions, starts, layer)
        ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, 3)      # the mma.sync kernel
        legacy = gpu_run(ctx, case, q, tables, positions, starts, layer)
        close(legacy, want)
        ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, 2)      # head_dim 64: the tcgen05 kernel
        tiled = gpu_run(ctx, case, q, tables, positions, starts, layer)
    finally:
        ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, 1)
    return per_entry, tiled, want


@pytest.mark.parametrize("hd,H,KH", [(64, 32, 4), (128, 32, 8), (64, 8, 8), (128, 8, 4), (64, 16, 4)])
def test_shared_table_chunk_of_consecutive_positions(ctx, oracle, hd, H, KH):
    """A prefill chunk: 70 consecutive positions (not a multiple of the row tile) starting inside a block, with and
    without a sliding window, on both layers of a two-layer pool."""
    pos = list(range(37, 107))
    for window, layer in ((None, 0), (50, 1), (1, 0)):
        st = [max(0, p + 1 - window) if window else 0 for p in pos]
        per_entry, tiled, want = shared_table_case(ctx, oracle, hd, H, KH, pos, st, 99, seed=hd + H + (window or 0), layers=2, layer=layer)
        close(tiled, want)
        close(tiled, per_entry)


def test_shared_table_long_context_many_tiles(ctx, oracle):
    """Windows that span many 64-token tiles, chunk at the end of a long context."""
    pos = list(range(1500, 1628))
    per_entry, tiled, want = shared_table_case(ctx, oracle, 64, 32, 4, pos, [0] * len(pos), 999, seed=3)
    close(tiled, want)
    close(tiled, per_entry)
    st = [max(0, p - 700) for p in pos]
    per_entry, tiled, want = shared_table_case(ctx, oracle, 128, 16, 4, pos, st, 999, seed=4)
    close(tiled, want)


def test_shared_table_unmapped_tail_empty_windows_and_scattered_positions(ctx, oracle):
    """Positions in arbitrary order; blocks past the mapped length score -inf (never read); a window that lies wholly in
    the unmapped tail or is empty gives zeros, not NaN."""
    rng = np.random.default_rng(8)
    pos = [int(p) for p in rng.integers(0, 200, 45)]
    st = [0] * 45
    st[3], pos[3] = 50, 49            # empty window
    st[7], pos[7] = 130, 180          # wholly past the 6 mapped blocks (96 tokens)
    st[11], pos[11] = 90, 120         # straddles the end of the mapping
    per_entry, tiled, want = shared_table_case(ctx, oracle, 64, 8, 2, pos, st, 6, seed=5)
    assert np.all(np.isfinite(tiled))
    close(tiled, want)
    close(tiled, per_entry)
    assert np.all(tiled[3] == 0.0) and np.all(tiled[7] == 0.0)
    # nothing mapped at all
    per_entry, tiled, want = shared_table_case(ctx, oracle, 64, 8, 2, pos, st, 0, seed=6)
    assert np.all(tiled == 0.0)


def test_shared_table_pool_garbage_outside_the_windows_is_never_used(ctx, oracle):
    """Slots past the highest position hold NaN (a block that was handed out but not filled yet): the result must not
    change, because those slots are neither scored nor multiplied."""
    from paged_infer_b200 import api
    hd, H, KH = 64, 32, 4
    pos = list(range(3, 75))
    case = AttnCase(H, KH, hd, 16, 1, 6, 6)
    case.kv_cache = normal_f32(case.kv_cache.size, 21, 1.0)
    q = normal_f32(len(pos) * H * hd, 22, 1.0)
    tables = [case.tables[0]] * len(pos)
    want = cpu_run(oracle, case, q, tables, pos, [0] * len(pos))
    kv = case.kv_cache.reshape(1, case.total_blocks, 16, KH, 2, hd)
    kv[0, case.tables[0][4], 11:, :, :, :] = np.nan     # tokens 75.. of the sequence
    kv[0, case.tables[0][5]] = np.nan
    for opt in (2, 3):
        ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, opt)
        try:
            got = gpu_run(ctx, case, q, tables, pos, [0] * len(pos))
        finally:
            ctx.set_option(api._lib.PI_OPT_ATTN_SHARED, 1)
        close(got, want)
