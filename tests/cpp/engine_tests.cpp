// The C++ engine loop (include/paged_infer_engine.hpp) on a small synthetic int8 model: requests with shared prompt
// prefixes, a two-sample request (fork + copy-on-write) and a tight KV pool, run to completion through the batched
// step; every request's greedy tokens must equal those of the same request run alone, from scratch, one token at a
// time in a fresh pool (the engine_tests.rs invariants: batching, prefix reuse and forking change no output).
#include <algorithm>
#include <cstdio>
#include <map>
#include <vector>

#include "../../include/paged_infer_engine.hpp"

#define CHECK(cond)                                                  \
  do {                                                               \
    if (!(cond)) {                                                   \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);  \
      return 1;                                                      \
    }                                                                \
  } while (0)
#define OK(call)                                                                   \
  do {                                                                             \
    if ((call) != PI_OK) {                                                         \
      std::printf("FAILED %s:%d: %s: %s\n", __FILE__, __LINE__, #call, pi_last_error(ctx)); \
      return 1;                                                                    \
    }                                                                              \
  } while (0)

static std::vector<uint32_t> alone(pi_ctx* ctx, pi_model* model, const pi_kv_layout& L1, const std::vector<uint32_t>& prompt, size_t max_tokens,
                                   bool* ok) {
  *ok = false;
  pi_kv_layout L = L1;
  L.block_size = 16;
  L.num_blocks = (int)((prompt.size() + max_tokens) / 16 + 2);
  pi_kv_pool* pool = nullptr;
  if (pi_kv_pool_create(ctx, &L, &pool) != PI_OK) return {};
  std::vector<int32_t> table;
  for (int i = 0; i < L.num_blocks; ++i) table.push_back(i);
  std::vector<uint32_t> out;
  uint32_t tok = 0;
  if (pi_model_prefill(ctx, model, pool, prompt.data(), (int)prompt.size(), 0, table.data(), (int)table.size(), 7, nullptr, &tok) != PI_OK) return {};
  out.push_back(tok);
  while (out.size() < max_tokens) {
    const int32_t pos = (int32_t)(prompt.size() + out.size() - 1), len = (int32_t)table.size();
    uint32_t next = 0;
    if (pi_model_decode_batch(ctx, model, pool, &tok, &pos, table.data(), len, &len, 1, nullptr, &next) != PI_OK) return {};
    out.push_back(next);
    tok = next;
  }
  pi_kv_pool_destroy(pool);
  *ok = true;
  return out;
}

int main() {
  pi_ctx* ctx = nullptr;
  if (pi_ctx_create(0, nullptr, &ctx) != PI_OK) {
    std::printf("FAILED pi_ctx_create: %s\n", pi_last_error(nullptr));
    return 1;
  }
  pi_model_config mc = {};
  mc.hidden_size = 256; mc.num_hidden_layers = 2; mc.num_attention_heads = 4; mc.num_key_value_heads = 2;
  mc.intermediate_size = 512; mc.vocab_size = 512; mc.rms_norm_eps = 1e-5f; mc.rope_theta = 10000.f;
  mc.attention_window = -1; mc.rope_style = 0; mc.max_batch = 32; mc.max_positions = 512;
  pi_model* model = nullptr;
  OK(pi_model_create_synthetic(ctx, &mc, 11, 0.05f, PI_INT8, PI_INT8, &model));
  pi_kv_layout L1 = {mc.num_hidden_layers, 1, 16, mc.num_key_value_heads, mc.hidden_size / mc.num_attention_heads};

  // prompts: three share a 40-token prefix (two full blocks), one is exactly two blocks long (fully cached on re-use)
  auto tokens = [](uint32_t seed, size_t n) {
    std::vector<uint32_t> v;
    uint32_t s = seed * 2654435761u + 12345u;
    for (size_t i = 0; i < n; ++i) { s = s * 1664525u + 1013904223u; v.push_back((s >> 9) % 512u); }
    return v;
  };
  const std::vector<uint32_t> prefix = tokens(1, 40);
  auto with_prefix = [&](uint32_t seed, size_t extra) { auto v = prefix; auto t = tokens(seed, extra); v.insert(v.end(), t.begin(), t.end()); return v; };
  std::vector<pi::Request> reqs;
  reqs.push_back({0, with_prefix(2, 9), 12, 1});
  reqs.push_back({1, with_prefix(3, 3), 20, 1});
  reqs.push_back({2, tokens(4, 32), 10, 1});
  reqs.push_back({3, tokens(5, 5), 25, 2});          // two samples: fork, then copy-on-write in the partial block
  reqs.push_back({4, with_prefix(6, 17), 8, 1});
  reqs.push_back({5, tokens(4, 32), 6, 1});          // same as request 2: the whole prompt comes out of the cache
  reqs.push_back({6, tokens(7, 70), 5, 1});

  pi::EngineConfig ec;
  ec.block_size = 16; ec.num_blocks = 40; ec.max_batch_size = 5; ec.prefill_chunk_size = 16;
  {
    pi::Engine eng(ctx, model, L1, ec);
    for (const auto& r : reqs) eng.add_request(r);
    std::map<uint64_t, std::vector<pi::Completion>> done;
    int guard = 0;
    while (eng.has_work() && ++guard < 400) {
      eng.step();
      for (auto& c : eng.take_finished()) done[c.request_id].push_back(std::move(c));
    }
    CHECK(!eng.has_work());
    CHECK(eng.memory().active_sequences() == 0);
    CHECK(eng.memory().cow_copies() >= 1);                         // the forked pair diverged inside a shared block
    CHECK(eng.memory().prefix_stats().hits >= 4);                   // the shared prefix and the repeated prompt
    CHECK(eng.stats().prompt_tokens_prefilled < eng.stats().prompt_tokens);
    for (const auto& r : reqs) {
      bool ok = false;
      const auto want = alone(ctx, model, L1, r.tokens, r.max_tokens, &ok);
      CHECK(ok);
      CHECK(done[r.id].size() == r.num_samples);
      for (const auto& c : done[r.id]) {
        CHECK(c.reason == pi::FinishReason::Length);
        CHECK(c.generated == want);
      }
    }
    CHECK(done[5][0].cached_prompt_tokens == 32);
    std::printf("steps %llu, decode batches %llu, prefilled %llu of %llu prompt tokens, cow copies %llu, cache hits %llu\n",
                (unsigned long long)eng.stats().steps, (unsigned long long)eng.stats().decode_batches,
                (unsigned long long)eng.stats().prompt_tokens_prefilled, (unsigned long long)eng.stats().prompt_tokens,
                (unsigned long long)eng.memory().cow_copies(), (unsigned long long)eng.memory().prefix_stats().hits);
  }
  {  // a pool too small for everything at once: requests wait for memory, none is lost; a sequence that cannot grow
     // ends with OutOfMemory (src/engine.rs:655-668) and what it produced until then is still the right prefix
    pi::EngineConfig tight = ec;
    tight.num_blocks = 9;
    pi::Engine eng(ctx, model, L1, tight);
    for (const auto& r : reqs) if (r.id != 6) eng.add_request(r);
    std::map<uint64_t, std::vector<pi::Completion>> done;
    int guard = 0;
    while (eng.has_work() && ++guard < 2000) {
      eng.step();
      for (auto& c : eng.take_finished()) done[c.request_id].push_back(std::move(c));
    }
    CHECK(!eng.has_work());
    size_t by_length = 0;
    for (const auto& r : reqs) {
      if (r.id == 6) continue;
      bool ok = false;
      const auto want = alone(ctx, model, L1, r.tokens, r.max_tokens, &ok);
      CHECK(ok && done[r.id].size() == r.num_samples);
      for (const auto& c : done[r.id]) {
        CHECK(c.reason == pi::FinishReason::Length || c.reason == pi::FinishReason::OutOfMemory);
        CHECK(c.generated.size() <= want.size() && std::equal(c.generated.begin(), c.generated.end(), want.begin()));
        if (c.reason == pi::FinishReason::Length) {
          CHECK(c.generated == want);
          ++by_length;
        }
      }
    }
    CHECK(by_length >= 3);
    CHECK(eng.memory().active_sequences() == 0);
  }
  pi_model_destroy(model);
  pi_ctx_destroy(ctx);
  std::printf("PASS\n");
  return 0;
}
