// C ABI over the host-side block bookkeeping of include/paged_infer_memory.hpp (BlockAllocator, PrefixCache,
// KvCacheManager: the C++ restatement of the reference's src/memory/*.rs), so that a host written in another
// language - here the Python benchmark and tests, in the reference the Rust engine itself - can drive the device
// library exactly as Engine::step does (src/engine.rs:496-586, :612-699): admit with the chained block hash ->
// prefill what the cache did not cover -> publish -> fork -> ensure_writable (copy-on-write) -> batched decode ->
// release.  Plain pointers and sizes only.  The shim keeps every live sequence's BlockTable; physical block ids
// are what the device library's block tables take.  Pure host code: no CUDA.
#include <cstdint>
#include <cstring>
#include <map>
#include <vector>

#include "../../include/paged_infer_memory.hpp"

using pi::mem::BlockTable;
using pi::mem::KvCacheManager;
using pi::mem::PhysicalBlock;

struct pih_manager {
  KvCacheManager kv;
  std::map<size_t, BlockTable> tables;
  pih_manager(size_t blocks, size_t bs) : kv(blocks, bs) {}
};

extern "C" {

pih_manager* pih_create(size_t num_blocks, size_t block_size, int prefix_cache) {
  if (num_blocks == 0 || block_size == 0) return nullptr;
  pih_manager* m = new pih_manager(num_blocks, block_size);
  m->kv.with_prefix_cache(prefix_cache != 0);
  return m;
}

void pih_destroy(pih_manager* m) { delete m; }

// KvCacheManager::admit (src/memory/kv_cache_manager.rs:116-200).  Returns the number of leading prompt tokens whose
// KV came from the prefix cache (prefill resumes there), or -1 when the pool cannot house the prompt.
long pih_admit(pih_manager* m, size_t seq_id, const uint32_t* tokens, size_t n, uint64_t tick) {
  std::vector<uint32_t> t(tokens, tokens + n);
  auto adm = m->kv.admit(seq_id, t, tick);
  if (!adm) return -1;
  m->tables[seq_id] = adm->block_table;
  return (long)adm->cached_tokens;
}

// publish_prompt_blocks (:214-233): offer the prompt blocks this sequence computed to the cache.
long pih_publish(pih_manager* m, size_t seq_id) {
  auto it = m->tables.find(seq_id);
  if (it == m->tables.end()) return -1;
  return (long)m->kv.publish_prompt_blocks(it->second);
}

// fork (:262-296): the child maps every block of the parent; nothing is copied.
int pih_fork(pih_manager* m, size_t parent_seq, size_t child_seq, uint64_t tick) {
  auto it = m->tables.find(parent_seq);
  if (it == m->tables.end() || m->tables.count(child_seq)) return -1;
  m->tables[child_seq] = m->kv.fork(it->second, child_seq, tick);
  return 0;
}

void pih_release(pih_manager* m, size_t seq_id) {
  m->kv.release_sequence(seq_id);
  m->tables.erase(seq_id);
}

// Length of the sequence's block table; the physical ids are written to `out` (up to `cap`).
long pih_table(pih_manager* m, size_t seq_id, int32_t* out, size_t cap) {
  auto it = m->tables.find(seq_id);
  if (it == m->tables.end()) return -1;
  const auto& slots = it->second.slots();
  for (size_t i = 0; i < slots.size() && i < cap; ++i) out[i] = (int32_t)slots[i].block;
  return (long)slots.size();
}

// What Engine::plan_step does before a batched forward (src/engine.rs:612-699) for B rows: sequence seq_ids[b] will
// write position positions[b].  Grows each mapping to cover the position, splits a shared block copy-on-write
// (ensure_writable, :298-327), and writes the final tables as one packed [B][width] int32 matrix (-1 padded) plus
// their lengths - the form the device library's decode call takes.  The (src, dst) pairs of the copies made go to
// cow_pairs ([2 * B] at most) for the caller to replay on the device pool BEFORE the forward.  Returns the number
// of copies, -1 when the pool is exhausted, -2 when a table is wider than `width`, -3 for an unknown sequence.
long pih_prepare_step(pih_manager* m, const uint64_t* seq_ids, const int32_t* positions, int B, uint64_t tick, int32_t* tables_out,
                      int width, int32_t* lens_out, int32_t* cow_pairs) {
  long copies = 0;
  const size_t bs = m->kv.block_size();
  for (int b = 0; b < B; ++b) {
    auto it = m->tables.find((size_t)seq_ids[b]);
    if (it == m->tables.end()) return -3;
    BlockTable& t = it->second;
    const size_t pos = (size_t)positions[b];
    const size_t needed = pos / bs + 1;
    while (t.len() < needed)
      if (!m->kv.append_block((size_t)seq_ids[b], t, tick)) return -1;
    const bool copied = m->kv.ensure_writable((size_t)seq_ids[b], t, pos, [&](PhysicalBlock src, PhysicalBlock dst) {
      cow_pairs[2 * copies] = (int32_t)src;
      cow_pairs[2 * copies + 1] = (int32_t)dst;
    });
    if (copied) ++copies;
    else if (m->kv.allocator().is_shared(t.slots()[pos / bs].block)) return -1;   // shared and no block left to split into
    m->kv.touch((size_t)seq_ids[b], tick);
    if ((int)t.len() > width) return -2;
    int32_t* row = tables_out + (size_t)b * width;
    const auto& slots = t.slots();
    for (size_t i = 0; i < slots.size(); ++i) row[i] = (int32_t)slots[i].block;
    for (int i = (int)slots.size(); i < width; ++i) row[i] = -1;
    lens_out[b] = (int32_t)slots.size();
  }
  return copies;
}

// out[0..7]: prefix-cache hits, misses, tokens saved, resident cache entries, copy-on-write copies, free blocks,
// total blocks, live sequences.
void pih_stats(const pih_manager* m, uint64_t* out) {
  const auto s = m->kv.prefix_stats();
  out[0] = s.hits;
  out[1] = s.misses;
  out[2] = s.tokens_saved;
  out[3] = 0;
  out[4] = m->kv.cow_copies();
  out[5] = m->kv.available_blocks();
  out[6] = m->kv.total_blocks();
  out[7] = m->kv.active_sequences();
}

}  // extern "C"
