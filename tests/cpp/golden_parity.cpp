// The reference's tests/golden_parity_tests.rs written against the C++ host mirror
// (include/paged_infer.hpp): a bf16 checkpoint in HuggingFace layout goes through the
// loader, the paged KV pool and the block table, and the logits must match the NumPy
// HF-Llama golden file within 5e-4 with zero argmax mismatches
// (tests/golden_parity_tests.rs:125-211).  Usage: golden_parity <fixture dir>
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>

#include "paged_infer.hpp"

static std::vector<char> slurp(const std::string& p) {
  std::ifstream f(p, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + p);
  return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

// Minimal safetensors reader: name -> (pointer to bf16 bits, rows, cols).
struct Checkpoint {
  std::vector<char> raw;
  std::string header;
  size_t base = 0;
  struct View { const uint16_t* data; long rows, cols; };
  explicit Checkpoint(const std::string& path) : raw(slurp(path)) {
    uint64_t hlen;
    memcpy(&hlen, raw.data(), 8);
    header.assign(raw.data() + 8, raw.data() + 8 + hlen);
    base = 8 + hlen;
  }
  View tensor(const std::string& name) const {
    const size_t at = header.find("\"" + name + "\":{");
    if (at == std::string::npos) throw std::runtime_error("missing tensor: " + name);
    auto list_after = [&](const char* key) {
      const size_t k = header.find(key, at), lb = header.find('[', k), rb = header.find(']', lb);
      std::vector<long> v;
      std::stringstream ss(header.substr(lb + 1, rb - lb - 1));
      for (std::string item; std::getline(ss, item, ',');) v.push_back(std::stol(item));
      return v;
    };
    const auto shape = list_after("\"shape\""), off = list_after("\"data_offsets\"");
    return {reinterpret_cast<const uint16_t*>(raw.data() + base + off[0]), shape[0], shape.size() > 1 ? shape[1] : 1};
  }
};

static float bf16(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }

static size_t argmax_last(const float* v, size_t n) {  // max_by(total_cmp): the last maximum wins
  size_t best = 0;
  for (size_t i = 1; i < n; ++i) if (v[i] >= v[best]) best = i;
  return best;
}

int main(int argc, char** argv) {
  try {
    const std::string dir = argc > 1 ? argv[1] : "tests/golden";
    std::map<std::string, std::string> meta;
    {
      std::ifstream f(dir + "/tiny_llama_meta.txt");
      for (std::string line; std::getline(f, line);) {
        const size_t eq = line.find('=');
        if (eq != std::string::npos) meta[line.substr(0, eq)] = line.substr(eq + 1);
      }
    }
    pi::LlamaConfig cfg;
    cfg.hidden_size = std::stoul(meta["hidden_size"]);
    cfg.num_hidden_layers = std::stoul(meta["num_hidden_layers"]);
    cfg.num_attention_heads = std::stoul(meta["num_attention_heads"]);
    cfg.num_key_value_heads = std::stoul(meta["num_key_value_heads"]);
    cfg.intermediate_size = std::stoul(meta["intermediate_size"]);
    cfg.vocab_size = std::stoul(meta["vocab_size"]);
    cfg.rms_norm_eps = std::stof(meta["rms_norm_eps"]);
    cfg.rope_theta = std::stof(meta["rope_theta"]);
    std::vector<uint32_t> tokens;
    {
      std::stringstream ss(meta["tokens"]);
      for (std::string t; std::getline(ss, t, ',');) tokens.push_back((uint32_t)std::stoul(t));
    }
    const auto graw = slurp(dir + "/tiny_llama_golden.bin");
    const float* golden = reinterpret_cast<const float*>(graw.data());
    const size_t V = cfg.vocab_size, NL = cfg.num_hidden_layers;

    // ModelLoader::load_weights (src/model.rs:398-446): Quantization::F32 keeps the bf16 checkpoint values.
    Checkpoint ck(dir + "/tiny_llama.safetensors");
    auto widen = [&](const std::string& name) {
      const auto v = ck.tensor(name);
      std::vector<float> out((size_t)v.rows * v.cols);
      for (size_t i = 0; i < out.size(); ++i) out[i] = bf16(v.data[i]);
      return out;
    };
    std::vector<std::vector<float>> norms;
    std::vector<const float*> attn_norm, ffn_norm;
    std::vector<pi_tensor> proj;
    const char* names[7] = {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                            "mlp.gate_proj", "mlp.down_proj", "mlp.up_proj"};
    norms.reserve(2 * NL + 1);
    for (size_t l = 0; l < NL; ++l) {
      const std::string p = "model.layers." + std::to_string(l) + ".";
      norms.push_back(widen(p + "input_layernorm.weight"));
      attn_norm.push_back(norms.back().data());
      norms.push_back(widen(p + "post_attention_layernorm.weight"));
      ffn_norm.push_back(norms.back().data());
      for (const char* n : names) {
        const auto v = ck.tensor(p + n + ".weight");
        proj.push_back(pi_tensor{PI_BF16, 0, v.rows, v.cols, v.data, nullptr});
      }
    }
    norms.push_back(widen("model.norm.weight"));
    const auto head = ck.tensor("lm_head.weight");
    pi_model_weights w{};
    w.token_embeddings_bf16 = ck.tensor("model.embed_tokens.weight").data;
    w.final_norm = norms.back().data();
    w.attention_norm = attn_norm.data();
    w.ffn_norm = ffn_norm.data();
    w.projections = proj.data();
    w.lm_head = pi_tensor{PI_BF16, 0, head.rows, head.cols, head.data, nullptr};

    pi::Context ctx(0);
    pi::LlamaWeights model(ctx, cfg, w, 64);
    const size_t BLOCK = 16, nblocks = (tokens.size() + BLOCK - 1) / BLOCK;
    auto compare = [&](const float* got, const float* want, size_t rows, const char* what) {
      float max_abs = 0.f;
      size_t mism = 0;
      for (size_t r = 0; r < rows; ++r) {
        for (size_t i = 0; i < V; ++i) max_abs = std::max(max_abs, std::fabs(got[r * V + i] - want[r * V + i]));
        mism += argmax_last(got + r * V, V) != argmax_last(want + r * V, V);
      }
      printf("%s: max|delta| %.3g, argmax mismatches %zu/%zu\n", what, max_abs, mism, rows);
      return max_abs < 5e-4f && mism == 0;
    };
    bool ok = true;
    {  // test_incremental_decode_matches_reference
      pi::KvCache kv(ctx, cfg.kv_layout(nblocks + 2, BLOCK));
      pi::BlockTable table;
      for (size_t i = 0; i < nblocks; ++i) table.append_block((int32_t)(nblocks + 1 - i));  // scattered
      std::vector<float> all;
      for (size_t i = 0; i < tokens.size(); ++i) {
        const auto logits = model.forward(tokens[i], i, table, kv);
        all.insert(all.end(), logits.begin(), logits.end());
      }
      ok &= compare(all.data(), golden, tokens.size(), "incremental decode");
    }
    {  // test_prefill_matches_reference_final_position + split prefill == whole
      pi::KvCache kv(ctx, cfg.kv_layout(nblocks, BLOCK)), kv2(ctx, cfg.kv_layout(nblocks, BLOCK));
      pi::BlockTable table;
      for (size_t i = 0; i < nblocks; ++i) table.append_block((int32_t)i);
      const auto whole = model.prefill_batched(tokens, 0, table, kv, 8);
      ok &= compare(whole.data(), golden + (tokens.size() - 1) * V, 1, "batched prefill, last position");
      std::vector<uint32_t> a(tokens.begin(), tokens.begin() + 23), b(tokens.begin() + 23, tokens.end());
      model.prefill(a, 0, table, kv2);
      const auto split = model.prefill(b, 23, table, kv2);
      float d = 0.f;
      for (size_t i = 0; i < V; ++i) d = std::max(d, std::fabs(split[i] - whole[i]));
      printf("split prefill vs whole: max|delta| %.3g\n", d);
      ok &= d < 1e-5f;
    }
    {  // the reference's shape assertions come back as errors, not aborts
      bool threw = false;
      try {
        pi::KvCache kv(ctx, cfg.kv_layout(1, BLOCK));
        pi::BlockTable t;
        t.append_block(0);
        model.prefill_batched({}, 0, t, kv, 4);
      } catch (const pi::Error& e) {
        threw = e.status == PI_ERR_INVALID_ARG;
      }
      ok &= threw;
    }
    puts(ok ? "PASS" : "FAIL");
    return ok ? 0 : 1;
  } catch (const std::exception& e) {
    fprintf(stderr, "error: %s\n", e.what());
    return 2;
  }
}
