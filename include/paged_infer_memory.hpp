// Host-side KV block bookkeeping of the engine, restated in C++17 (header only, no CUDA dependency):
// the reference's BlockAllocator (src/memory/allocator.rs:16-111), BlockSlot / BlockTable
// (src/memory/block_table.rs:5-93), PrefixCache with its chained FNV-1a block hash
// (src/memory/prefix_cache.rs:28-199) and KvCacheManager (src/memory/kv_cache_manager.rs:38-404).
// Pure integer logic: which physical block a sequence maps, who holds references, what is shared, what
// is evicted.  The one place that touches KV data - cloning a shared block before a write - goes
// through a callback, which on the device is pi_kv_copy_block (stream-ordered ahead of the step).
//
// Where the Rust code asserts, these throw std::logic_error with the same message.
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace pi {
namespace mem {

using PhysicalBlock = int32_t;

// Reference-counted pool of physical blocks; a block returns to the free list with its last reference.
class BlockAllocator {
 public:
  BlockAllocator(size_t total_blocks, size_t block_size) : block_size(block_size), refs_(total_blocks, 0) {
    for (size_t i = 0; i < total_blocks; ++i) free_.push_back((PhysicalBlock)i);
  }
  size_t block_size;

  std::optional<PhysicalBlock> allocate() {   // first-in first-out over the free list, one reference
    if (free_.empty()) return std::nullopt;
    const PhysicalBlock b = free_.front();
    free_.pop_front();
    refs_[b] = 1;
    return b;
  }
  void incref(PhysicalBlock b) {
    check(b);
    if (refs_[b] == 0) throw std::logic_error("incref on a free block (index " + std::to_string(b) + ")");
    ++refs_[b];
  }
  bool free(PhysicalBlock b) {   // true when this was the last reference
    check(b);
    if (refs_[b] == 0) throw std::logic_error("double free of block " + std::to_string(b));
    if (--refs_[b] == 0) {
      free_.push_back(b);
      return true;
    }
    return false;
  }
  uint32_t ref_count(PhysicalBlock b) const {
    check(b);
    return refs_[b];
  }
  bool is_shared(PhysicalBlock b) const { return ref_count(b) > 1; }
  size_t available_blocks() const { return free_.size(); }
  size_t total_blocks() const { return refs_.size(); }
  size_t allocated_blocks() const { return refs_.size() - free_.size(); }

 private:
  void check(PhysicalBlock b) const {
    if (b < 0 || (size_t)b >= refs_.size())
      throw std::logic_error("physical block index " + std::to_string(b) + " out of range (total " + std::to_string(refs_.size()) + ")");
  }
  std::deque<PhysicalBlock> free_;
  std::vector<uint32_t> refs_;
};

// One logical block of a sequence: the physical block, the hash of the whole prefix up to and including it
// (complete prompt blocks only) and whether its KV came out of the prefix cache.
struct BlockSlot {
  PhysicalBlock block = -1;
  std::optional<uint64_t> hash;
  bool cached = false;
};

class BlockTable {
 public:
  void append_block(PhysicalBlock b) { slots_.push_back(BlockSlot{b, std::nullopt, false}); }
  void append_slot(const BlockSlot& s) { slots_.push_back(s); }
  // (block, offset) of a token, or nullopt past the mapping
  std::optional<std::pair<PhysicalBlock, size_t>> get_physical_location(size_t token, size_t block_size) const {
    const size_t lb = token / block_size;
    if (lb >= slots_.size()) return std::nullopt;
    return std::make_pair(slots_[lb].block, token % block_size);
  }
  const std::vector<BlockSlot>& slots() const { return slots_; }
  std::vector<BlockSlot>& slots_mut() { return slots_; }
  std::vector<PhysicalBlock> physical_blocks() const {
    std::vector<PhysicalBlock> v;
    for (const auto& s : slots_) v.push_back(s.block);
    return v;
  }
  size_t len() const { return slots_.size(); }
  bool is_empty() const { return slots_.empty(); }
  // Point a logical block at a fresh private copy: it is no longer the cached block, and has no stable hash.
  void remap(size_t logical, PhysicalBlock b) {
    BlockSlot& s = slots_.at(logical);
    s.block = b;
    s.hash.reset();
    s.cached = false;
  }

 private:
  std::vector<BlockSlot> slots_;
};

constexpr uint64_t kRootHash = 0;

// FNV-1a over the previous block's hash followed by this block's tokens (little-endian bytes), with the
// token count folded in, so that a block's key depends on its entire prefix.
inline uint64_t block_hash(uint64_t parent, const uint32_t* tokens, size_t n) {
  constexpr uint64_t kPrime = 0x00000100000001B3ull;
  uint64_t h = parent ^ 0xcbf29ce484222325ull;
  for (size_t i = 0; i < n; ++i)
    for (int b = 0; b < 4; ++b) {
      h ^= (uint64_t)((tokens[i] >> (8 * b)) & 0xFFu);
      h *= kPrime;
    }
  h ^= (uint64_t)n;
  return h * kPrime;
}

struct PrefixCacheStats {
  uint64_t hits = 0, misses = 0, inserts = 0, evictions = 0, tokens_saved = 0;
  double hit_rate() const { return hits + misses == 0 ? 0.0 : (double)hits / (double)(hits + misses); }
};

// prefix hash -> physical block holding that prefix's KV.  The cache holds one reference per stored block.
class PrefixCache {
 public:
  std::optional<PhysicalBlock> lookup(uint64_t hash) {   // the caller increfs before mapping the block
    ++tick_;
    auto it = entries_.find(hash);
    if (it == entries_.end()) {
      ++stats_.misses;
      return std::nullopt;
    }
    it->second.last_used = tick_;
    ++stats_.hits;
    return it->second.block;
  }
  void insert(uint64_t hash, PhysicalBlock block, BlockAllocator& alloc) {   // a second insert of a hash is a no-op
    if (entries_.count(hash)) return;
    ++tick_;
    alloc.incref(block);
    entries_[hash] = Entry{block, tick_};
    ++stats_.inserts;
  }
  // Drop the least recently used entry whose block nobody else maps.
  bool evict_lru(BlockAllocator& alloc) {
    auto victim = entries_.end();
    for (auto it = entries_.begin(); it != entries_.end(); ++it)
      if (alloc.ref_count(it->second.block) == 1 && (victim == entries_.end() || it->second.last_used < victim->second.last_used))
        victim = it;
    if (victim == entries_.end()) return false;
    alloc.free(victim->second.block);
    entries_.erase(victim);
    ++stats_.evictions;
    return true;
  }
  bool evict_until_available(BlockAllocator& alloc, size_t wanted) {
    while (alloc.available_blocks() < wanted)
      if (!evict_lru(alloc)) return false;
    return true;
  }
  void clear(BlockAllocator& alloc) {
    for (auto& kv : entries_) {
      alloc.free(kv.second.block);
      ++stats_.evictions;
    }
    entries_.clear();
  }
  size_t len() const { return entries_.size(); }
  bool is_empty() const { return entries_.empty(); }
  PrefixCacheStats stats() const { return stats_; }
  void reset_stats() { stats_ = PrefixCacheStats{}; }
  void record_tokens_saved(size_t tokens) { stats_.tokens_saved += tokens; }

 private:
  struct Entry {
    PhysicalBlock block;
    uint64_t last_used;
  };
  std::unordered_map<uint64_t, Entry> entries_;
  uint64_t tick_ = 0;
  PrefixCacheStats stats_;
};

struct Admission {
  BlockTable block_table;
  size_t cached_tokens = 0;     // leading prompt tokens whose KV came from the cache: prefill starts here
  size_t reused_blocks = 0;
  size_t allocated_blocks = 0;
};

// Sequence-level ownership of KV blocks: prefix reuse at admission, copy-on-write before a write into a
// shared block, eviction of cold cache entries (then of the least recently used sequence) under pressure.
class KvCacheManager {
 public:
  // Clones physical block `src` into `dst` across all layers (KvLayout::copy_block / pi_kv_copy_block).
  using CopyBlock = std::function<void(PhysicalBlock src, PhysicalBlock dst)>;

  KvCacheManager(size_t total_blocks, size_t block_size) : alloc_(total_blocks, block_size) {}
  KvCacheManager& with_prefix_cache(bool enabled) {
    cache_enabled_ = enabled;
    return *this;
  }
  size_t block_size() const { return alloc_.block_size; }
  size_t available_blocks() const { return alloc_.available_blocks(); }
  size_t total_blocks() const { return alloc_.total_blocks(); }
  const BlockAllocator& allocator() const { return alloc_; }
  PrefixCacheStats prefix_stats() const { return cache_.stats(); }
  uint64_t cow_copies() const { return cow_copies_; }
  size_t active_sequences() const { return seqs_.size(); }

  void clear() {   // back to the initial state, counters included
    std::vector<size_t> ids;
    for (auto& kv : seqs_) ids.push_back(kv.first);
    for (size_t id : ids) release_sequence(id);
    cache_.clear(alloc_);
    cache_.reset_stats();
    cow_copies_ = 0;
  }

  // Map blocks for a prompt, reusing cached KV for its longest known prefix; nullopt when the prompt cannot be
  // housed even after evicting cold cache entries (the rejected admission leaves no references behind).
  std::optional<Admission> admit(size_t seq_id, const std::vector<uint32_t>& tokens, uint64_t now_tick) {
    const size_t bs = alloc_.block_size;
    const size_t total = std::max<size_t>((tokens.size() + bs - 1) / bs, 1);
    const size_t full = tokens.size() / bs;          // a trailing partial block has no stable identity yet
    std::vector<uint64_t> hashes;
    uint64_t parent = kRootHash;
    for (size_t b = 0; b < full; ++b) {
      parent = block_hash(parent, tokens.data() + b * bs, bs);
      hashes.push_back(parent);
    }
    Admission adm;
    size_t reused = 0;
    if (cache_enabled_)
      for (uint64_t h : hashes) {                      // stop at the first miss: later blocks have another history
        const auto hit = cache_.lookup(h);
        if (!hit) break;
        alloc_.incref(*hit);
        adm.block_table.append_slot(BlockSlot{*hit, h, true});
        ++reused;
      }
    const size_t to_allocate = total - reused;
    if (alloc_.available_blocks() < to_allocate && !cache_.evict_until_available(alloc_, to_allocate)) {
      for (const auto& s : adm.block_table.slots()) alloc_.free(s.block);
      return std::nullopt;
    }
    for (size_t i = reused; i < total; ++i) {
      const auto b = alloc_.allocate();
      if (!b) throw std::logic_error("capacity was just verified");
      adm.block_table.append_slot(BlockSlot{*b, i < hashes.size() ? std::optional<uint64_t>(hashes[i]) : std::nullopt, false});
    }
    adm.cached_tokens = reused * bs;
    adm.reused_blocks = reused;
    adm.allocated_blocks = to_allocate;
    cache_.record_tokens_saved(adm.cached_tokens);
    seqs_[seq_id] = SequenceAlloc{adm.block_table.physical_blocks(), now_tick};
    return adm;
  }

  // Publish the prompt blocks this sequence computed (hash known, not themselves cache hits); returns how many
  // entries were added.
  size_t publish_prompt_blocks(const BlockTable& table) {
    if (!cache_enabled_) return 0;
    size_t published = 0;
    for (const auto& s : table.slots())
      if (s.hash && !s.cached) {
        const size_t before = cache_.len();
        cache_.insert(*s.hash, s.block, alloc_);
        published += cache_.len() - before;
      }
    return published;
  }

  // One more block for a sequence that has run past the end of its mapping.
  bool append_block(size_t seq_id, BlockTable& table, uint64_t now_tick) {
    touch(seq_id, now_tick);
    if (alloc_.available_blocks() == 0 && !cache_.evict_until_available(alloc_, 1)) return false;
    const auto b = alloc_.allocate();
    if (!b) return false;
    table.append_block(*b);
    auto it = seqs_.find(seq_id);
    if (it == seqs_.end()) it = seqs_.emplace(seq_id, SequenceAlloc{{}, now_tick}).first;
    it->second.blocks.push_back(*b);
    return true;
  }

  // The child maps every one of the parent's blocks; no data moves.
  BlockTable fork(const BlockTable& parent, size_t child_seq, uint64_t now_tick) {
    BlockTable child;
    for (const auto& s : parent.slots()) {
      alloc_.incref(s.block);
      child.append_slot(s);
    }
    seqs_[child_seq] = SequenceAlloc{child.physical_blocks(), now_tick};
    return child;
  }

  // Make the block holding `token_pos` privately writable; true if a copy was made.
  bool ensure_writable(size_t seq_id, BlockTable& table, size_t token_pos, const CopyBlock& copy_block) {
    const size_t logical = token_pos / alloc_.block_size;
    if (logical >= table.len()) return false;
    const PhysicalBlock old = table.slots()[logical].block;
    if (!alloc_.is_shared(old)) return false;
    if (alloc_.available_blocks() == 0 && !cache_.evict_until_available(alloc_, 1)) return false;   // caller must preempt
    const auto fresh = alloc_.allocate();
    if (!fresh) return false;
    copy_block(old, *fresh);
    table.remap(logical, *fresh);
    alloc_.free(old);
    auto it = seqs_.find(seq_id);
    if (it != seqs_.end()) {
      auto pos = std::find(it->second.blocks.begin(), it->second.blocks.end(), old);
      if (pos != it->second.blocks.end()) *pos = *fresh;
    }
    ++cow_copies_;
    return true;
  }

  void touch(size_t seq_id, uint64_t now_tick) {
    auto it = seqs_.find(seq_id);
    if (it != seqs_.end()) it->second.last_used_tick = now_tick;
  }

  // Drop a sequence's references; blocks the prefix cache still holds stay resident.
  void release_sequence(size_t seq_id) {
    auto it = seqs_.find(seq_id);
    if (it == seqs_.end()) return;
    for (PhysicalBlock b : it->second.blocks) alloc_.free(b);
    seqs_.erase(it);
  }

  // Single-block path of the eviction benchmark: one block for a sequence, giving up a cold cache entry first and
  // (if allowed) the least recently used other sequence last.  Among equally old sequences the lowest id goes.
  bool ensure_block_for_sequence(size_t seq_id, uint64_t now_tick, bool allow_eviction) {
    touch(seq_id, now_tick);
    if (const auto b = alloc_.allocate()) return record(seq_id, *b, now_tick);
    if (cache_.evict_lru(alloc_))
      if (const auto b = alloc_.allocate()) return record(seq_id, *b, now_tick);
    if (!allow_eviction) return false;
    bool found = false;
    size_t victim = 0;
    uint64_t oldest = 0;
    for (const auto& kv : seqs_)
      if (kv.first != seq_id && (!found || kv.second.last_used_tick < oldest)) {
        found = true;
        victim = kv.first;
        oldest = kv.second.last_used_tick;
      }
    if (found) {
      release_sequence(victim);
      if (const auto b = alloc_.allocate()) return record(seq_id, *b, now_tick);
    }
    return false;
  }

 private:
  struct SequenceAlloc {
    std::vector<PhysicalBlock> blocks;
    uint64_t last_used_tick;
  };
  bool record(size_t seq_id, PhysicalBlock b, uint64_t now_tick) {
    auto it = seqs_.find(seq_id);
    if (it == seqs_.end()) it = seqs_.emplace(seq_id, SequenceAlloc{{}, now_tick}).first;
    it->second.blocks.push_back(b);
    return true;
  }
  BlockAllocator alloc_;
  std::map<size_t, SequenceAlloc> seqs_;
  PrefixCache cache_;
  bool cache_enabled_ = true;
  uint64_t cow_copies_ = 0;
};

}  // namespace mem
}  // namespace pi
