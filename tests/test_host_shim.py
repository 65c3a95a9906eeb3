"""The C ABI over the host-side block bookkeeping (``libpaged_infer_host.so``, ``paged_infer_b200/host.py``):
the scenario the benchmark drives - prompts that share a prefix, published blocks found by later admissions through
the chained hash, a fork, the copy-on-write split on the first write, growth across a block boundary - checked
against the rules of the reference's KvCacheManager (src/memory/kv_cache_manager.rs:116-345).  No GPU."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def host():
    from paged_infer_b200 import build, host
    build.build_host()
    return host


def test_library_exports_every_declared_symbol(host):
    L = host.lib()
    for name in host.SIGNATURES:
        assert hasattr(L, name), name


def test_prefix_reuse_fork_and_copy_on_write(host):
    BS = 16
    m = host.KvCacheManager(64, BS)
    rng = np.random.default_rng(0)
    prefix = rng.integers(0, 1000, 40).astype(np.uint32)          # two full blocks + 8 tokens
    a = np.concatenate([prefix, rng.integers(0, 1000, 9).astype(np.uint32)])
    b = np.concatenate([prefix, rng.integers(0, 1000, 30).astype(np.uint32)])
    assert m.admit(1, a) == 0                                      # nothing cached yet
    assert m.publish_prompt_blocks(1) == 3                         # 49 tokens: three full blocks get an identity
    assert m.admit(2, b) == 2 * BS                                 # the two blocks of the common prefix are found
    ta, tb = m.table(1), m.table(2)
    assert ta[:2] == tb[:2] and ta[2] != tb[2] and len(ta) == 4 and len(tb) == 5
    m.fork(1, 3)
    assert m.table(3) == ta
    # first write after the fork: position 49 lies in the shared partial block -> one split, for whoever goes first
    ids = np.array([1, 3, 2], np.uint64)
    pos = np.array([49, 49, 70], np.int32)
    tables = np.empty((3, 8), np.int32)
    lens = np.empty(3, np.int32)
    cow = np.empty((3, 2), np.int32)
    assert m.prepare_step(ids, pos, tables, lens, cow) == 1
    assert cow[0, 0] == ta[3] and cow[0, 1] == tables[0, 3] and tables[1, 3] == ta[3]
    assert lens.tolist() == [4, 4, 5] and tables[0, :3].tolist() == ta[:3] and (tables[:, 5:] == -1).all()
    assert m.prepare_step(ids, pos + 1, tables, lens, cow) == 0    # private now
    # growth across a block boundary
    pos2 = np.array([64, 64, 80], np.int32)
    assert m.prepare_step(ids, pos2, tables, lens, cow) == 0
    assert lens.tolist() == [5, 5, 6]
    st = m.stats()
    assert st["cow_copies"] == 1 and st["prefix_hits"] == 2 and st["prefix_tokens_saved"] == 32 and st["live_sequences"] == 3
    m.release_sequence(3)
    m.release_sequence(1)
    m.release_sequence(2)
    st = m.stats()
    assert st["live_sequences"] == 0 and st["free_blocks"] == 64 - 3   # the cache still holds the three published blocks


def test_out_of_blocks_is_reported_not_hidden(host):
    m = host.KvCacheManager(2, 16, prefix_cache=False)
    m.admit(1, np.arange(20, dtype=np.uint32))
    with pytest.raises(host.OutOfBlocks):
        m.admit(2, np.arange(5, dtype=np.uint32))
    ids, pos = np.array([1], np.uint64), np.array([32], np.int32)
    with pytest.raises(host.OutOfBlocks):
        m.prepare_step(ids, pos, np.empty((1, 4), np.int32), np.empty(1, np.int32), np.empty((1, 2), np.int32))
