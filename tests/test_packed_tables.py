"""PackedBlockTables (host arrays updated in place) must always equal the flattening of the same tables."""
import numpy as np


def test_packed_tables_follow_appends_and_remaps():
    from paged_infer_b200 import api
    rng = np.random.default_rng(0)
    tables = [[int(x) for x in rng.integers(0, 1000, n)] for n in (3, 0, 7, 1)]
    pk = api.PackedBlockTables(len(tables), 4)
    for b, t in enumerate(tables):
        pk.set_row(b, t)
    for step in range(50):
        b = int(rng.integers(0, len(tables)))
        if tables[b] and rng.random() < 0.3:
            i = int(rng.integers(0, len(tables[b])))
            tables[b][i] = 2000 + step
            pk.remap(b, i, 2000 + step)
        else:
            tables[b].append(3000 + step)
            pk.append(b, 3000 + step)
        want_mat, want_lens, want_mb = api.pack_block_tables(tables)
        mat, lens, mb = api.pack_block_tables(pk)
        assert mb == want_mb and np.array_equal(lens, want_lens) and np.array_equal(mat, want_mat)
    pk.set_row(2, [5])
    tables[2] = [5]
    want_mat, want_lens, want_mb = api.pack_block_tables(tables)
    mat, lens, mb = api.pack_block_tables(pk)
    assert mb == want_mb and np.array_equal(lens, want_lens) and np.array_equal(mat, want_mat)
