// The engine's step loop over the device library, restated in C++17 (header only): what Engine::step does in the
// reference (src/engine.rs:485-839) with greedy sampling and no speculation -
//
//   admit    waiting requests while the KV pool can house them: map the longest cached prefix, prefill only what
//            the cache did not cover (the last prompt token is always recomputed for its logits), publish the
//            prompt's blocks, fork extra samples (src/engine.rs:496-586)
//   decode   settle memory for every live sequence first (grow the mapping, split shared blocks copy-on-write:
//            src/engine.rs:612-699), then advance all of them with ONE batched call and commit the chosen tokens
//   reclaim  release finished sequences (their cached prompt blocks stay resident for later requests)
//
// The KV pool lives on the device (pi_kv_pool), block bookkeeping is pi::mem::KvCacheManager, the forward passes are
// pi_model_prefill / pi_model_decode_batch with the greedy choice made on the device (only token ids come back).
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <vector>

#include "paged_infer_cuda.h"
#include "paged_infer_memory.hpp"

namespace pi {

struct EngineConfig {
  size_t block_size = 16;
  size_t num_blocks = 256;
  size_t max_batch_size = 64;        // rows of one batched forward (BatchScratch capacity, src/engine.rs:210); more live
                                     // sequences than this are advanced in several passes per step
  size_t prefill_chunk_size = 32;
  uint32_t eos_token = 0xFFFFFFFFu;
  bool prefix_cache = true;
};

enum class FinishReason { None, Eos, Length, OutOfMemory };

struct Request {
  uint64_t id = 0;
  std::vector<uint32_t> tokens;
  size_t max_tokens = 16;
  size_t num_samples = 1;
};

struct Completion {
  uint64_t request_id = 0;
  size_t sequence_id = 0;
  std::vector<uint32_t> generated;
  FinishReason reason = FinishReason::None;
  size_t cached_prompt_tokens = 0;
};

struct EngineStats {
  uint64_t steps = 0, requests = 0, prompt_tokens = 0, prompt_tokens_prefilled = 0, generated_tokens = 0, decode_batches = 0;
};

class EngineError : public std::runtime_error {
 public:
  explicit EngineError(const std::string& m) : std::runtime_error(m) {}
};

class Engine {
 public:
  // `ctx` and `model` stay owned by the caller; the engine owns the KV pool.
  Engine(pi_ctx* ctx, pi_model* model, const pi_kv_layout& layout_one_block, const EngineConfig& cfg)
      : ctx_(ctx), model_(model), cfg_(cfg), kv_(cfg.num_blocks, cfg.block_size) {
    kv_.with_prefix_cache(cfg.prefix_cache);
    if (cfg_.max_batch_size == 0) throw EngineError("max_batch_size must be at least 1");
    // one batched forward never exceeds what the model's scratch was built for
    const int cap = pi_model_max_batch(model_);
    if (cap > 0 && (size_t)cap < cfg_.max_batch_size) cfg_.max_batch_size = (size_t)cap;
    pi_kv_layout L = layout_one_block;
    L.num_blocks = (int)cfg.num_blocks;
    L.block_size = (int)cfg.block_size;
    check(pi_kv_pool_create(ctx_, &L, &pool_), "pi_kv_pool_create");
  }
  ~Engine() {
    if (pool_) pi_kv_pool_destroy(pool_);
  }
  Engine(const Engine&) = delete;
  Engine& operator=(const Engine&) = delete;

  void add_request(Request r) {
    if (r.tokens.empty()) throw EngineError("a request needs at least one prompt token");
    if (r.num_samples == 0) r.num_samples = 1;
    waiting_.push_back(std::move(r));
  }
  bool has_work() const { return !waiting_.empty() || !active_.empty(); }
  size_t active_sequences() const { return active_.size(); }
  const EngineStats& stats() const { return stats_; }
  const mem::KvCacheManager& memory() const { return kv_; }
  std::vector<Completion> take_finished() {
    std::vector<Completion> out;
    out.swap(finished_);
    return out;
  }

  void step() {
    ++tick_;
    admit();
    decode();
    reclaim();
    ++stats_.steps;
  }

 private:
  struct Sequence {
    size_t id = 0;
    uint64_t request_id = 0;
    std::vector<uint32_t> token_ids;   // prompt + generated
    std::vector<uint32_t> generated;
    size_t max_tokens = 0;
    size_t cached_prompt_tokens = 0;
    mem::BlockTable table;
    FinishReason finished = FinishReason::None;
  };

  void check(pi_status s, const char* what) {
    if (s != PI_OK) throw EngineError(std::string(what) + ": " + pi_last_error(ctx_));
  }
  static std::vector<int32_t> ids_of(const mem::BlockTable& t) {
    std::vector<int32_t> v;
    for (const auto& s : t.slots()) v.push_back(s.block);
    return v;
  }

  void admit() {
    // Memory is the only gate, as in the reference (src/engine.rs:496-503): a request is admitted as soon as the pool
    // can house its prompt; the number of live sequences is not limited here (decode() advances them in passes).
    // All samples of one request are decoded greedily and therefore identical; the reference gives such requests a
    // temperature of 0.8 (src/engine.rs:543-551), and sampling beyond argmax stays with the host
    // (pi_model_decode_batch_rows hands back the logits of the sequences that need it).
    while (!waiting_.empty()) {
      const Request& req = waiting_.front();
      const size_t seq_id = next_seq_++;
      auto adm = kv_.admit(seq_id, req.tokens, tick_);
      if (!adm) {
        --next_seq_;
        break;   // out of memory even after reclaiming cold cache blocks: wait for a live sequence to retire
      }
      // replay only what the cache did not cover; a fully cached prompt still recomputes its last token for the logits
      const size_t resume_at = std::min(adm->cached_tokens, req.tokens.size() - 1);
      const std::vector<int32_t> ids = ids_of(adm->block_table);
      uint32_t first = 0;
      check(pi_model_prefill(ctx_, model_, pool_, req.tokens.data() + resume_at, (int)(req.tokens.size() - resume_at), (int)resume_at,
                             ids.data(), (int)ids.size(), (int)cfg_.prefill_chunk_size, nullptr, &first),
            "pi_model_prefill");
      ++stats_.requests;
      stats_.prompt_tokens += req.tokens.size();
      stats_.prompt_tokens_prefilled += req.tokens.size() - resume_at;
      kv_.publish_prompt_blocks(adm->block_table);

      std::vector<std::pair<size_t, mem::BlockTable>> tables;
      tables.emplace_back(seq_id, adm->block_table);
      for (size_t i = 1; i < req.num_samples; ++i) {   // extra samples map the parent's blocks; divergence is paid lazily
        const size_t child = next_seq_++;
        tables.emplace_back(child, kv_.fork(tables[0].second, child, tick_));
      }
      for (auto& st : tables) {
        Sequence s;
        s.id = st.first;
        s.request_id = req.id;
        s.token_ids = req.tokens;
        s.token_ids.push_back(first);
        s.generated = {first};
        s.max_tokens = req.max_tokens;
        s.cached_prompt_tokens = adm->cached_tokens;
        s.table = std::move(st.second);
        if (first == cfg_.eos_token) s.finished = FinishReason::Eos;
        else if (req.max_tokens <= 1) s.finished = FinishReason::Length;
        ++stats_.generated_tokens;
        active_.push_back(std::move(s));
      }
      waiting_.pop_front();
    }
  }

  void decode() {
    // settle memory first: the batched forward needs the block tables final
    std::vector<size_t> run;
    for (size_t idx = 0; idx < active_.size(); ++idx) {
      Sequence& s = active_[idx];
      if (s.finished != FinishReason::None) continue;
      const size_t pos = s.token_ids.size() - 1;
      const size_t needed = (pos + 1 + cfg_.block_size - 1) / cfg_.block_size;
      bool oom = false;
      while (s.table.len() < needed)
        if (!kv_.append_block(s.id, s.table, tick_)) {
          oom = true;
          break;
        }
      if (oom && s.table.len() * cfg_.block_size <= pos) {
        s.finished = FinishReason::OutOfMemory;
        continue;
      }
      // forked siblings map the same partial block: split before writing
      kv_.ensure_writable(s.id, s.table, pos, [&](mem::PhysicalBlock src, mem::PhysicalBlock dst) {
        check(pi_kv_copy_block(ctx_, pool_, src, dst), "pi_kv_copy_block");
      });
      kv_.touch(s.id, tick_);
      run.push_back(idx);
    }
    if (run.empty()) return;

    // passes of at most max_batch_size rows, like run_groups (src/engine.rs:722-760)
    for (size_t start = 0; start < run.size(); start += cfg_.max_batch_size) {
      const int B = (int)std::min(cfg_.max_batch_size, run.size() - start);
      size_t max_blocks = 1;
      for (int b = 0; b < B; ++b) max_blocks = std::max(max_blocks, active_[run[start + b]].table.len());
      std::vector<uint32_t> tokens(B), chosen(B);
      std::vector<int32_t> positions(B), lens(B), tables((size_t)B * max_blocks, -1);
      for (int b = 0; b < B; ++b) {
        const Sequence& s = active_[run[start + b]];
        tokens[b] = s.token_ids.back();
        positions[b] = (int32_t)(s.token_ids.size() - 1);
        lens[b] = (int32_t)s.table.len();
        for (size_t i = 0; i < s.table.len(); ++i) tables[(size_t)b * max_blocks + i] = s.table.slots()[i].block;
      }
      check(pi_model_decode_batch(ctx_, model_, pool_, tokens.data(), positions.data(), tables.data(), (int)max_blocks, lens.data(), B,
                                  nullptr, chosen.data()),
            "pi_model_decode_batch");
      ++stats_.decode_batches;
      for (int b = 0; b < B; ++b) {   // commit
        Sequence& s = active_[run[start + b]];
        s.token_ids.push_back(chosen[b]);
        s.generated.push_back(chosen[b]);
        ++stats_.generated_tokens;
        if (chosen[b] == cfg_.eos_token) s.finished = FinishReason::Eos;
        else if (s.generated.size() >= s.max_tokens) s.finished = FinishReason::Length;
      }
    }
  }

  void reclaim() {
    std::vector<Sequence> keep;
    for (auto& s : active_) {
      if (s.finished == FinishReason::None) {
        keep.push_back(std::move(s));
        continue;
      }
      kv_.release_sequence(s.id);
      Completion c;
      c.request_id = s.request_id;
      c.sequence_id = s.id;
      c.generated = std::move(s.generated);
      c.reason = s.finished;
      c.cached_prompt_tokens = s.cached_prompt_tokens;
      finished_.push_back(std::move(c));
    }
    active_.swap(keep);
  }

  pi_ctx* ctx_;
  pi_model* model_;
  EngineConfig cfg_;
  mem::KvCacheManager kv_;
  pi_kv_pool* pool_ = nullptr;
  std::deque<Request> waiting_;
  std::vector<Sequence> active_;
  std::vector<Completion> finished_;
  EngineStats stats_;
  uint64_t tick_ = 0;
  size_t next_seq_ = 0;
};

}  // namespace pi
