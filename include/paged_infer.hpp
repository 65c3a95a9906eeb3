// paged_infer.hpp - header-only C++17 host mirror of the reference's Rust interface
// for the decode hot path, over the C ABI of libpaged_infer_cuda.so.
//
// Type and method names follow the reference crate (src/model.rs, src/attention.rs,
// src/memory/layout.rs, src/memory/block_table.rs, src/math.rs, src/sampling.rs); where
// the Rust code asserts or panics these throw pi::Error carrying the library's status
// and message.  Host vectors in, host vectors out; weights, KV pool and scratch live on
// the device inside the handles.  Nothing here computes on the CPU.
#pragma once

#include <algorithm>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "paged_infer_cuda.h"

namespace pi {

struct Error : std::runtime_error {
  pi_status status;
  Error(pi_status s, const std::string& m) : std::runtime_error("paged_infer_cuda error " + std::to_string(s) + ": " + m), status(s) {}
};

inline void check(pi_status s, const pi_ctx* ctx) {
  if (s != PI_OK) throw Error(s, pi_last_error(ctx));
}

// One device, one stream, one host thread.
class Context {
 public:
  explicit Context(int device = 0, void* stream = nullptr) {
    check(pi_ctx_create(device, stream, &ctx_), nullptr);
  }
  Context(int device, void* stream, int rank, int tp, const void* nccl_id) {
    check(pi_ctx_create_tp(device, stream, rank, tp, nccl_id, &ctx_), nullptr);
  }
  ~Context() { pi_ctx_destroy(ctx_); }
  Context(const Context&) = delete;
  Context& operator=(const Context&) = delete;
  pi_ctx* get() const { return ctx_; }
  void synchronize() { check(pi_ctx_synchronize(ctx_), ctx_); }

 private:
  pi_ctx* ctx_ = nullptr;
};

// math::quantize_rows_i8 (src/math.rs:456-469): (codes, scales).
inline std::pair<std::vector<int8_t>, std::vector<float>> quantize_rows_i8(Context& c, const std::vector<float>& w, size_t rows, size_t cols) {
  if (w.size() != rows * cols) throw Error(PI_ERR_INVALID_ARG, "weight length != rows * cols");
  std::vector<int8_t> q(rows * cols);
  std::vector<float> s(rows);
  check(pi_quantize_rows_i8(c.get(), w.data(), rows, cols, q.data(), s.data()), c.get());
  return {std::move(q), std::move(s)};
}

// sampling::argmax (src/sampling.rs:140-147): ties go to the last index.
inline uint32_t argmax(Context& c, const std::vector<float>& logits) {
  uint32_t out = 0;
  check(pi_argmax_host(c.get(), logits.data(), 1, (int)logits.size(), &out), c.get());
  return out;
}

// Projection::{F32, Int8} (src/model.rs:218-291).
class Projection {
 public:
  // QuantizedLinear {rows, cols, weight, scales}
  static Projection int8(Context& c, size_t rows, size_t cols, const int8_t* q, const float* scales) {
    pi_linear* l = nullptr;
    check(pi_linear_create_i8(c.get(), rows, cols, q, scales, PI_SPLIT_NONE, &l), c.get());
    return Projection(c, l);
  }
  // QuantizedLinear::from_packed
  static Projection from_packed(Context& c, size_t rows, size_t cols, const float* w) {
    pi_linear* l = nullptr;
    check(pi_linear_create_quantized(c.get(), rows, cols, w, PI_SPLIT_NONE, &l), c.get());
    return Projection(c, l);
  }
  // PackedLinear from bf16 checkpoint bits
  static Projection bf16(Context& c, size_t rows, size_t cols, const uint16_t* w) {
    pi_linear* l = nullptr;
    check(pi_linear_create_bf16(c.get(), rows, cols, w, PI_SPLIT_NONE, &l), c.get());
    return Projection(c, l);
  }
  static Projection f32(Context& c, size_t rows, size_t cols, const float* w) {
    pi_linear* l = nullptr;
    check(pi_linear_create_f32(c.get(), rows, cols, w, PI_SPLIT_NONE, &l), c.get());
    return Projection(c, l);
  }
  size_t rows() const { return pi_linear_rows(l_.get()); }
  size_t cols() const { return pi_linear_cols(l_.get()); }
  size_t weight_bytes() const { return pi_linear_weight_bytes(l_.get()); }
  // apply_parallel: one activation vector
  std::vector<float> apply_parallel(const std::vector<float>& x) const { return apply_batched(x, 1); }
  // apply_batched: x_br [batch][cols] -> [batch][rows]
  std::vector<float> apply_batched(const std::vector<float>& x_br, int batch) const {
    if (batch < 1 || x_br.size() != (size_t)batch * cols()) throw Error(PI_ERR_INVALID_ARG, "x_br must hold batch * cols elements");
    std::vector<float> out((size_t)batch * rows());
    check(pi_linear_apply_host(c_->get(), l_.get(), x_br.data(), out.data(), batch), c_->get());
    return out;
  }

 private:
  Projection(Context& c, pi_linear* l) : c_(&c), l_(l, pi_linear_destroy) {}
  Context* c_;
  std::shared_ptr<pi_linear> l_;
};
using QuantizedLinear = Projection;
using PackedLinear = Projection;

// KvLayout (src/memory/layout.rs:18-97): the reference's address arithmetic.
struct KvLayout {
  size_t num_layers, num_blocks, block_size, num_kv_heads, head_dim;
  size_t total_floats() const { return num_layers * num_blocks * block_stride(); }
  size_t block_stride() const { return block_size * num_kv_heads * 2 * head_dim; }
  size_t index(size_t layer, size_t phys_block, size_t token_offset, size_t kv_head, bool is_value) const {
    return ((((layer * num_blocks + phys_block) * block_size + token_offset) * num_kv_heads + kv_head) * 2 + (is_value ? 1 : 0)) * head_dim;
  }
};

// BlockTable (src/memory/block_table.rs:28-93).
struct BlockTable {
  std::vector<int32_t> logical_to_physical;
  void append_block(int32_t b) { logical_to_physical.push_back(b); }
  size_t len() const { return logical_to_physical.size(); }
  // Some((block, offset)) or none (first < 0)
  std::pair<int32_t, size_t> get_physical_location(size_t logical_token_idx, size_t block_size) const {
    const size_t lb = logical_token_idx / block_size;
    if (lb >= logical_to_physical.size()) return {-1, 0};
    return {logical_to_physical[lb], logical_token_idx % block_size};
  }
  void remap(size_t logical_block_idx, int32_t b) { logical_to_physical.at(logical_block_idx) = b; }
};

// The engine's kv_cache (src/engine.rs:206-207), resident on the device.
class KvCache {
 public:
  KvCache(Context& c, const KvLayout& l) : c_(&c), layout_(l) {
    const pi_kv_layout cl{(int32_t)l.num_layers, (int32_t)l.num_blocks, (int32_t)l.block_size, (int32_t)l.num_kv_heads, (int32_t)l.head_dim};
    pi_kv_pool* p = nullptr;
    check(pi_kv_pool_create(c.get(), &cl, &p), c.get());
    pool_.reset(p, pi_kv_pool_destroy);
  }
  const KvLayout& layout() const { return layout_; }
  pi_kv_pool* get() const { return pool_.get(); }
  void copy_block(int32_t src, int32_t dst) { check(pi_kv_copy_block(c_->get(), pool_.get(), src, dst), c_->get()); }  // KvLayout::copy_block
  void upload(const std::vector<float>& cache) {
    if (cache.size() != layout_.total_floats()) throw Error(PI_ERR_INVALID_ARG, "cache length does not match the layout");
    check(pi_kv_upload(c_->get(), pool_.get(), cache.data()), c_->get());
  }
  std::vector<float> download() const {
    std::vector<float> out(layout_.total_floats());
    check(pi_kv_download(c_->get(), pool_.get(), out.data()), c_->get());
    return out;
  }

 private:
  Context* c_;
  KvLayout layout_;
  std::shared_ptr<pi_kv_pool> pool_;
};

// AttnEntry (src/attention.rs:58-85)
struct AttnEntry {
  const BlockTable* block_table;
  size_t pos, start;
  AttnEntry(const BlockTable& t, size_t pos_, long window = -1)
      : block_table(&t), pos(pos_), start(window < 0 ? 0 : (pos_ + 1 > (size_t)window ? pos_ + 1 - (size_t)window : 0)) {}
  size_t window_len() const { return pos + 1 > start ? pos + 1 - start : 0; }
};

inline void pack_tables(const std::vector<const BlockTable*>& tables, std::vector<int32_t>& mat, std::vector<int32_t>& lens, int& max_blocks) {
  max_blocks = 0;
  for (auto* t : tables) max_blocks = std::max(max_blocks, (int)t->len());
  const int mb = std::max(max_blocks, 1);
  mat.assign(tables.size() * mb, -1);
  lens.resize(tables.size());
  for (size_t b = 0; b < tables.size(); ++b) {
    lens[b] = (int32_t)tables[b]->len();
    for (size_t i = 0; i < tables[b]->len(); ++i) mat[b * mb + i] = tables[b]->logical_to_physical[i];
  }
}

// PagedAttention::run (src/attention.rs:141-265): out [entries][num_heads][head_dim].
struct PagedAttention {
  KvLayout layout;
  size_t num_heads;
  std::vector<float> run(Context& c, const std::vector<float>& q, const KvCache& kv, const std::vector<AttnEntry>& entries, size_t layer) const {
    const size_t B = entries.size();
    if (q.size() != B * num_heads * layout.head_dim) throw Error(PI_ERR_INVALID_ARG, "q must be [entries][num_heads][head_dim]");
    std::vector<float> out(q.size(), 0.f);
    if (B == 0) return out;
    std::vector<const BlockTable*> tabs;
    std::vector<int32_t> pos, start, mat, lens;
    for (auto& e : entries) {
      tabs.push_back(e.block_table);
      pos.push_back((int32_t)e.pos);
      start.push_back((int32_t)e.start);
    }
    int mb = 0;
    pack_tables(tabs, mat, lens, mb);
    check(pi_paged_attention_host(c.get(), kv.get(), (int)layer, (int)num_heads, q.data(), out.data(), mat.data(), mb, lens.data(),
                                  pos.data(), start.data(), (int)B), c.get());
    return out;
  }
};

// LlamaConfig (src/model.rs:14-53)
struct LlamaConfig {
  size_t hidden_size = 2048, num_hidden_layers = 22, num_attention_heads = 32, num_key_value_heads = 4;
  size_t intermediate_size = 5632, vocab_size = 32000;
  float rms_norm_eps = 1e-5f, rope_theta = 10000.0f;
  long attention_window = -1;  // None
  int rope_style = 0;          // RopeStyle::Neox
  size_t head_dim() const { return hidden_size / num_attention_heads; }
  size_t kv_dim() const { return num_key_value_heads * head_dim(); }
  KvLayout kv_layout(size_t num_blocks, size_t block_size) const { return {num_hidden_layers, num_blocks, block_size, num_key_value_heads, head_dim()}; }
};

// LlamaWeights + forward entry points (src/model.rs:380-386, :585-1255).
class LlamaWeights {
 public:
  LlamaWeights(Context& c, const LlamaConfig& cfg, const pi_model_weights& w, int max_batch = 32, int max_positions = 4096)
      : c_(&c), cfg_(cfg) {
    pi_model_config mc{(int32_t)cfg.hidden_size, (int32_t)cfg.num_hidden_layers, (int32_t)cfg.num_attention_heads,
                       (int32_t)cfg.num_key_value_heads, (int32_t)cfg.intermediate_size, (int32_t)cfg.vocab_size,
                       cfg.rms_norm_eps, cfg.rope_theta, (int32_t)cfg.attention_window, cfg.rope_style, max_batch, max_positions};
    pi_model* m = nullptr;
    check(pi_model_create(c.get(), &mc, &w, &m), c.get());
    m_.reset(m, pi_model_destroy);
  }
  size_t weight_bytes() const { return pi_model_weight_bytes(m_.get()); }
  // forward: one token at `pos`, logits over the vocabulary
  std::vector<float> forward(uint32_t token_id, size_t pos, const BlockTable& table, KvCache& kv) {
    return decode_batch_into({token_id}, {pos}, {&table}, kv);
  }
  // decode_batch_into: logits [batch][vocab]
  std::vector<float> decode_batch_into(const std::vector<uint32_t>& tokens, const std::vector<size_t>& positions,
                                       const std::vector<const BlockTable*>& tables, KvCache& kv) {
    const size_t B = tokens.size();
    if (positions.size() != B || tables.size() != B) throw Error(PI_ERR_INVALID_ARG, "one position and one block table per token");
    std::vector<int32_t> pos(positions.begin(), positions.end()), mat, lens;
    int mb = 0;
    pack_tables(tables, mat, lens, mb);
    std::vector<float> logits(B * cfg_.vocab_size);
    check(pi_model_decode_batch(c_->get(), m_.get(), kv.get(), tokens.data(), pos.data(), mat.data(), mb, lens.data(), (int)B,
                                logits.data(), nullptr), c_->get());
    return logits;
  }
  // prefill_batched: logits of the last prompt position
  std::vector<float> prefill_batched(const std::vector<uint32_t>& tokens, size_t start_pos, const BlockTable& table, KvCache& kv, size_t chunk_size) {
    std::vector<float> logits(cfg_.vocab_size);
    check(pi_model_prefill(c_->get(), m_.get(), kv.get(), tokens.data(), (int)tokens.size(), (int)start_pos,
                           table.logical_to_physical.data(), (int)table.len(), (int)chunk_size, logits.data(), nullptr), c_->get());
    return logits;
  }
  std::vector<float> prefill(const std::vector<uint32_t>& tokens, size_t start_pos, const BlockTable& table, KvCache& kv) {
    return prefill_batched(tokens, start_pos, table, kv, 1);
  }

 private:
  Context* c_;
  LlamaConfig cfg_;
  std::shared_ptr<pi_model> m_;
};

}  // namespace pi
