// The engine loop (include/paged_infer_engine.hpp) over a FAKE of the device library: the handful of C-ABI calls the
// engine makes are defined here on the host, so the scheduling logic runs without a GPU.  The fake "model" maps
// (last token, position) to the next token with a fixed formula, checks every argument the engine passes (batch
// rows within the model's capacity, block tables long enough for the position, distinct writable blocks after a
// copy-on-write) and records the batch sizes it saw.
//
// Scenarios (reference behaviour: Engine::admit src/engine.rs:496-586, run_groups :702-760):
//   oversize      a request with more samples than max_batch_size is admitted (memory is the only gate) and finishes
//   capacity      max_batch_size above the model's scratch capacity: every forward stays within the capacity
//   passes        more live sequences than max_batch_size: several passes per step, every sequence advances once
//   queue         a request that does not fit the pool waits without blocking the step loop from draining the others
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "../../include/paged_infer_engine.hpp"

struct pi_ctx { std::string err; };
struct pi_model { int capacity; };
struct pi_kv_pool { pi_kv_layout L; std::vector<int> copies; };

static std::vector<int> g_batches;        // rows of every batched forward
static int g_prefills = 0, g_cow = 0;
static bool g_violation = false;

static uint32_t next_token(uint32_t tok, int pos) { return (tok * 31u + (uint32_t)pos * 7u + 3u) % 997u; }

extern "C" {
const char* pi_last_error(const pi_ctx* c) { return c ? c->err.c_str() : ""; }
int pi_model_max_batch(const pi_model* m) { return m->capacity; }
pi_status pi_kv_pool_create(pi_ctx*, const pi_kv_layout* L, pi_kv_pool** out) {
  *out = new pi_kv_pool{*L, {}};
  return PI_OK;
}
void pi_kv_pool_destroy(pi_kv_pool* p) { delete p; }
pi_status pi_kv_copy_block(pi_ctx* c, pi_kv_pool* p, int32_t src, int32_t dst) {
  if (src == dst || src < 0 || dst < 0 || src >= p->L.num_blocks || dst >= p->L.num_blocks) {
    c->err = "bad copy";
    return PI_ERR_INVALID_ARG;
  }
  ++g_cow;
  return PI_OK;
}
pi_status pi_model_prefill(pi_ctx*, pi_model*, pi_kv_pool* pool, const uint32_t* tokens, int n, int start_pos, const int32_t*,
                           int table_len, int, float*, uint32_t* argmax) {
  if (n < 1 || (start_pos + n + pool->L.block_size - 1) / pool->L.block_size > table_len) g_violation = true;
  ++g_prefills;
  if (argmax) *argmax = next_token(tokens[n - 1], start_pos + n - 1);
  return PI_OK;
}
pi_status pi_model_decode_batch(pi_ctx* c, pi_model* m, pi_kv_pool* pool, const uint32_t* tokens, const int32_t* positions,
                                const int32_t* tables, int max_blocks, const int32_t* lens, int B, float*, uint32_t* argmax) {
  if (B > m->capacity) {
    c->err = "batch exceeds scratch capacity";
    return PI_ERR_INVALID_ARG;
  }
  g_batches.push_back(B);
  std::set<int32_t> written;
  for (int b = 0; b < B; ++b) {
    const int lb = positions[b] / pool->L.block_size;
    if (lb >= lens[b] || lens[b] > max_blocks) g_violation = true;
    else if (!written.insert(tables[(size_t)b * max_blocks + lb]).second) g_violation = true;   // two rows write one block
    argmax[b] = next_token(tokens[b], positions[b]);
  }
  return PI_OK;
}
}

#define CHECK(cond)                                                  \
  do {                                                               \
    if (!(cond)) {                                                   \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);  \
      return 1;                                                      \
    }                                                                \
  } while (0)

static std::vector<uint32_t> prompt(uint32_t seed, size_t n) {
  std::vector<uint32_t> v;
  for (size_t i = 0; i < n; ++i) v.push_back((seed * 131u + (uint32_t)i * 17u) % 997u);
  return v;
}

static std::vector<uint32_t> expected(const std::vector<uint32_t>& p, size_t max_tokens) {
  std::vector<uint32_t> out;
  uint32_t tok = p.back();
  int pos = (int)p.size() - 1;
  while (out.size() < max_tokens) {
    tok = next_token(tok, pos++);
    out.push_back(tok);
  }
  return out;
}

static int run_all(pi::Engine& e, size_t want, std::map<uint64_t, std::vector<pi::Completion>>* done, int max_steps = 2000) {
  size_t got = 0;
  for (int s = 0; s < max_steps && e.has_work(); ++s) {
    e.step();
    for (auto& c : e.take_finished()) {
      (*done)[c.request_id].push_back(c);
      ++got;
    }
  }
  return (got == want && !e.has_work()) ? 0 : 1;
}

int main() {
  pi_ctx ctx;
  const pi_kv_layout L1 = {2, 1, 16, 2, 64};

  {  // oversize: 6 samples, max_batch_size 4 -> admitted, advanced in two passes per step, all complete
    g_batches.clear();
    pi_model model{64};
    pi::EngineConfig cfg;
    cfg.num_blocks = 64;
    cfg.max_batch_size = 4;
    pi::Engine e(&ctx, &model, L1, cfg);
    e.add_request({7, prompt(1, 20), 5, 6});
    e.add_request({8, prompt(2, 9), 3, 1});        // queued behind it: must not starve
    std::map<uint64_t, std::vector<pi::Completion>> done;
    CHECK(run_all(e, 7, &done) == 0);
    CHECK(done[7].size() == 6 && done[8].size() == 1);
    for (auto& c : done[7]) CHECK(c.generated == expected(prompt(1, 20), 5) && c.reason == pi::FinishReason::Length);
    CHECK(done[8][0].generated == expected(prompt(2, 9), 3));
    CHECK(*std::max_element(g_batches.begin(), g_batches.end()) <= 4);
    CHECK(g_cow >= 5);                             // the six siblings split their shared partial block
    std::printf("ok oversize\n");
  }
  {  // capacity: the engine is configured for 32 rows, the model's scratch holds 3
    g_batches.clear();
    pi_model model{3};
    pi::EngineConfig cfg;
    cfg.num_blocks = 64;
    cfg.max_batch_size = 32;
    pi::Engine e(&ctx, &model, L1, cfg);
    for (uint64_t r = 0; r < 8; ++r) e.add_request({r, prompt(10 + (uint32_t)r, 5 + r), 4, 1});
    std::map<uint64_t, std::vector<pi::Completion>> done;
    CHECK(run_all(e, 8, &done) == 0);
    for (uint64_t r = 0; r < 8; ++r) CHECK(done[r].size() == 1 && done[r][0].generated == expected(prompt(10 + (uint32_t)r, 5 + r), 4));
    CHECK(!g_batches.empty() && *std::max_element(g_batches.begin(), g_batches.end()) == 3);
    std::printf("ok capacity\n");
  }
  {  // passes: 10 live sequences, 4 rows per forward -> 3 forwards per step (4 + 4 + 2), every sequence advances once per step
    g_batches.clear();
    pi_model model{64};
    pi::EngineConfig cfg;
    cfg.num_blocks = 128;
    cfg.max_batch_size = 4;
    pi::Engine e(&ctx, &model, L1, cfg);
    for (uint64_t r = 0; r < 10; ++r) e.add_request({r, prompt(30 + (uint32_t)r, 18), 6, 1});
    e.step();
    CHECK(e.active_sequences() == 10);
    CHECK(g_batches.size() == 3 && g_batches[0] == 4 && g_batches[1] == 4 && g_batches[2] == 2);
    CHECK(e.stats().generated_tokens == 20);       // one token from each prefill, one from the step's decode
    std::map<uint64_t, std::vector<pi::Completion>> done;
    CHECK(run_all(e, 10, &done) == 0);
    for (uint64_t r = 0; r < 10; ++r) CHECK(done[r][0].generated == expected(prompt(30 + (uint32_t)r, 18), 6));
    std::printf("ok passes\n");
  }
  {  // queue: a prompt that needs more blocks than are free waits; the loop keeps draining the admitted ones
    pi_model model{64};
    pi::EngineConfig cfg;
    cfg.num_blocks = 6;
    cfg.max_batch_size = 8;
    cfg.prefix_cache = false;
    pi::Engine e(&ctx, &model, L1, cfg);
    e.add_request({1, prompt(50, 60), 3, 1});       // 4 blocks
    e.add_request({2, prompt(51, 60), 3, 1});       // 4 more: does not fit until request 1 retires
    e.step();
    CHECK(e.active_sequences() == 1);
    std::map<uint64_t, std::vector<pi::Completion>> done;
    CHECK(run_all(e, 2, &done) == 0);
    CHECK(done[1][0].generated == expected(prompt(50, 60), 3) && done[2][0].generated == expected(prompt(51, 60), 3));
    std::printf("ok queue\n");
  }
  bool threw = false;
  try {
    pi_model model{8};
    pi::EngineConfig cfg;
    cfg.max_batch_size = 0;
    pi::Engine e(&ctx, &model, L1, cfg);
  } catch (const pi::EngineError&) {
    threw = true;
  }
  CHECK(threw);
  CHECK(!g_violation);
  std::printf("all ok\n");
  return 0;
}
