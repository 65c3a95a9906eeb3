// Behaviour of the host-side KV block bookkeeping (include/paged_infer_memory.hpp), following the scenarios of the
// reference's unit tests (src/memory/kv_cache_manager.rs:418-636, src/memory/allocator.rs tests): prefix reuse,
// divergence, cache survival, eviction under pressure, rejected admissions, fork + copy-on-write, release order,
// churn.  Prints one "ok <name>" line per scenario and "hash <hex>" lines that the Python side checks against its
// own FNV-1a.  Exit code 0 only if every check held.
#include <cstdio>
#include <numeric>
#include <vector>

#include "../../include/paged_infer_memory.hpp"

using namespace pi::mem;

static int failures = 0;
#define CHECK(cond)                                                         \
  do {                                                                      \
    if (!(cond)) {                                                          \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);         \
      ++failures;                                                           \
    }                                                                       \
  } while (0)

static std::vector<uint32_t> seq(uint32_t from, uint32_t to) {
  std::vector<uint32_t> v;
  for (uint32_t i = from; i < to; ++i) v.push_back(i);
  return v;
}
static std::vector<uint32_t> cat(std::vector<uint32_t> a, const std::vector<uint32_t>& b) {
  a.insert(a.end(), b.begin(), b.end());
  return a;
}

constexpr size_t BS = 4;

int main() {
  {  // allocator: FIFO free list, reference counts, asserts
    BlockAllocator a(3, 16);
    auto b0 = a.allocate(), b1 = a.allocate(), b2 = a.allocate();
    CHECK(b0 && b1 && b2 && *b0 == 0 && *b1 == 1 && *b2 == 2 && !a.allocate());
    a.incref(*b1);
    CHECK(a.is_shared(*b1) && !a.is_shared(*b0) && a.ref_count(*b1) == 2);
    CHECK(!a.free(*b1) && a.free(*b1) && a.available_blocks() == 1);
    CHECK(a.free(*b0) && *a.allocate() == 1 && *a.allocate() == 0);   // freed blocks queue up behind
    bool threw = false;
    try { a.free(2); a.free(2); } catch (const std::logic_error&) { threw = true; }
    CHECK(threw);
    threw = false;
    try { a.incref(7); } catch (const std::logic_error&) { threw = true; }
    CHECK(threw);
    std::printf("ok allocator\n");
  }
  {  // block table
    BlockTable t;
    t.append_block(5);
    t.append_slot(BlockSlot{9, 123u, true});
    CHECK(t.len() == 2 && t.get_physical_location(5, 4)->first == 9 && t.get_physical_location(5, 4)->second == 1);
    CHECK(!t.get_physical_location(8, 4));
    t.remap(1, 3);
    CHECK(t.slots()[1].block == 3 && !t.slots()[1].hash && !t.slots()[1].cached);
    std::printf("ok block_table\n");
  }
  {  // hashes for the Python cross-check
    const std::vector<uint32_t> a = {0, 1, 2, 3}, b = {4, 5, 6, 7}, c = {0xFFFFFFFFu, 0x01020304u, 7};
    const uint64_t h1 = block_hash(kRootHash, a.data(), a.size());
    const uint64_t h2 = block_hash(h1, b.data(), b.size());
    std::printf("hash %016llx\nhash %016llx\nhash %016llx\nhash %016llx\n", (unsigned long long)h1, (unsigned long long)h2,
                (unsigned long long)block_hash(kRootHash, c.data(), c.size()), (unsigned long long)block_hash(kRootHash, nullptr, 0));
    CHECK(h1 != h2 && block_hash(kRootHash, b.data(), 4) != h2);   // chained: same tokens, other history
  }
  {  // single-block path with LRU preemption of a sequence
    KvCacheManager m(2, 16);
    CHECK(m.ensure_block_for_sequence(1, 1, false) && m.ensure_block_for_sequence(2, 2, false));
    CHECK(!m.ensure_block_for_sequence(3, 3, false));
    CHECK(m.ensure_block_for_sequence(3, 4, true) && m.active_sequences() == 2);
    std::printf("ok lru_preemption\n");
  }
  {  // the second request reuses the shared prefix
    KvCacheManager m(32, BS);
    const auto shared = seq(0, 12);
    auto a = m.admit(1, cat(shared, {90, 91}), 1);
    CHECK(a && a->reused_blocks == 0 && a->cached_tokens == 0 && a->allocated_blocks == 4);
    CHECK(m.publish_prompt_blocks(a->block_table) == 3);
    auto b = m.admit(2, cat(shared, {80, 81}), 2);
    CHECK(b && b->reused_blocks == 3 && b->cached_tokens == 12 && b->allocated_blocks == 1);
    for (int i = 0; i < 3; ++i) CHECK(a->block_table.slots()[i].block == b->block_table.slots()[i].block && b->block_table.slots()[i].cached);
    CHECK(a->block_table.slots()[3].block != b->block_table.slots()[3].block && !b->block_table.slots()[3].hash);
    CHECK(m.prefix_stats().tokens_saved == 12 && m.prefix_stats().hits == 3);
    CHECK(m.publish_prompt_blocks(b->block_table) == 0);   // hits are not re-published
    std::printf("ok prefix_reuse\n");
  }
  {  // reuse stops at the first divergent block
    KvCacheManager m(32, BS);
    auto a = m.admit(1, seq(0, 12), 1);
    m.publish_prompt_blocks(a->block_table);
    auto b = m.admit(2, {0, 1, 2, 3, 40, 41, 42, 43, 8, 9, 10, 11}, 2);
    CHECK(b && b->reused_blocks == 1 && a->block_table.slots()[2].block != b->block_table.slots()[2].block);
    std::printf("ok divergence\n");
  }
  {  // disabling the cache removes all reuse
    KvCacheManager m(32, BS);
    m.with_prefix_cache(false);
    auto a = m.admit(1, seq(0, 12), 1);
    CHECK(m.publish_prompt_blocks(a->block_table) == 0);
    auto b = m.admit(2, seq(0, 12), 2);
    CHECK(b && b->reused_blocks == 0 && b->allocated_blocks == 3);
    std::printf("ok cache_disabled\n");
  }
  {  // cached blocks survive their producer
    KvCacheManager m(8, BS);
    auto a = m.admit(1, seq(0, 8), 1);
    m.publish_prompt_blocks(a->block_table);
    m.release_sequence(1);
    CHECK(m.available_blocks() == 6);
    auto b = m.admit(2, seq(0, 8), 2);
    CHECK(b && b->reused_blocks == 2);
    std::printf("ok cache_survives\n");
  }
  {  // admission under pressure evicts the cache before failing
    KvCacheManager m(4, BS);
    auto a = m.admit(1, seq(0, 8), 1);
    m.publish_prompt_blocks(a->block_table);
    m.release_sequence(1);
    CHECK(m.available_blocks() == 2);
    auto b = m.admit(2, seq(90, 106), 2);
    CHECK(b.has_value() && m.prefix_stats().evictions >= 2);
    std::printf("ok eviction_under_pressure\n");
  }
  {  // a rejected admission leaves no references behind
    KvCacheManager m(4, BS);
    auto a = m.admit(1, seq(0, 8), 1);
    m.publish_prompt_blocks(a->block_table);
    const size_t before = m.available_blocks();
    CHECK(!m.admit(2, cat(seq(0, 8), seq(200, 240)), 2));
    CHECK(m.available_blocks() == before);
    for (const auto& s : a->block_table.slots()) CHECK(m.allocator().ref_count(s.block) == 2);   // sequence + cache
    auto c = m.admit(3, seq(0, 8), 3);
    CHECK(c && c->reused_blocks == 2);
    std::printf("ok rejected_admission\n");
  }
  {  // fork shares blocks and copies on write
    std::vector<std::pair<int, int>> copies;
    auto copy = [&](PhysicalBlock s, PhysicalBlock d) { copies.push_back({s, d}); };
    KvCacheManager m(8, BS);
    auto parent = m.admit(1, {1, 2, 3, 4, 5, 6}, 1);
    BlockTable pt = parent->block_table;
    CHECK(pt.len() == 2);
    const size_t before = m.available_blocks();
    BlockTable ct = m.fork(pt, 2, 2);
    CHECK(m.available_blocks() == before && ct.slots()[1].block == pt.slots()[1].block);
    CHECK(m.ensure_writable(2, ct, 6, copy));
    CHECK(ct.slots()[1].block != pt.slots()[1].block && m.cow_copies() == 1);
    CHECK(copies.size() == 1 && copies[0].first == pt.slots()[1].block && copies[0].second == ct.slots()[1].block);
    CHECK(ct.slots()[0].block == pt.slots()[0].block);              // the full block is still shared
    CHECK(!m.ensure_writable(2, ct, 6, copy) && m.cow_copies() == 1);   // private now
    CHECK(!m.ensure_writable(2, ct, 100, copy));                    // past the mapping
    m.release_sequence(2);
    m.release_sequence(1);
    CHECK(m.available_blocks() == m.total_blocks());                 // the clone was tracked by the child
    std::printf("ok fork_cow\n");
  }
  {  // an unshared block is never copied
    KvCacheManager m(8, BS);
    auto a = m.admit(1, {1, 2, 3}, 1);
    BlockTable t = a->block_table;
    int n = 0;
    CHECK(!m.ensure_writable(1, t, 2, [&](PhysicalBlock, PhysicalBlock) { ++n; }) && n == 0 && m.cow_copies() == 0);
    std::printf("ok unshared\n");
  }
  {  // copy-on-write against the cache's reference, with no free block: the cold cache entry gives way
    KvCacheManager m(2, BS);
    auto a = m.admit(1, seq(0, 4), 1);          // one full block
    m.publish_prompt_blocks(a->block_table);      // shared with the cache now
    BlockTable t = a->block_table;
    int n = 0;
    CHECK(m.available_blocks() == 1);
    CHECK(m.ensure_writable(1, t, 3, [&](PhysicalBlock, PhysicalBlock) { ++n; }) && n == 1);
    CHECK(m.append_block(1, t, 2) == true);       // last free block ... the cache entry (now unshared) is evicted for it
    CHECK(m.append_block(1, t, 3) == false);      // nothing left
    std::printf("ok cow_vs_cache\n");
  }
  {  // release after fork frees only the last holder
    KvCacheManager m(8, BS);
    auto p = m.admit(1, {1, 2, 3, 4}, 1);
    const size_t after = m.available_blocks();
    m.fork(p->block_table, 2, 2);
    m.release_sequence(1);
    CHECK(m.available_blocks() == after);
    m.release_sequence(2);
    CHECK(m.available_blocks() == m.total_blocks());
    std::printf("ok release_order\n");
  }
  {  // churn returns every block
    KvCacheManager m(64, BS);
    for (size_t round = 0; round < 500; ++round) {
      std::vector<uint32_t> unique;
      for (uint32_t i = 0; i < 4; ++i) unique.push_back((uint32_t)(round * 10 + i));
      auto a = m.admit(round, cat(seq(0, 8), unique), round);
      CHECK(a.has_value());
      if (!a) break;
      m.publish_prompt_blocks(a->block_table);
      m.release_sequence(round);
    }
    CHECK(m.active_sequences() == 0);
    m.clear();
    CHECK(m.available_blocks() == 64 && m.prefix_stats().hits == 0 && m.cow_copies() == 0);
    std::printf("ok churn\n");
  }
  std::printf(failures ? "FAILURES %d\n" : "all ok\n", failures);
  return failures ? 1 : 0;
}
