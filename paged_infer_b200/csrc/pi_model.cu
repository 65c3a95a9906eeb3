// Model forward on the device: the counterpart of LlamaWeights::run_layers_batch,
// decode_batch_into and prefill_batched (reference src/model.rs:968-1255).
//
// Per layer the reference's op order is kept - RMSNorm, q/k/v projections,
// rotary on q then k, K/V scatter for ALL entries, attention, o projection +
// residual, RMSNorm, gate/up, SwiGLU, down projection + residual - but fused
// into six kernels:
//   1. [q;k;v] projection with the RMSNorm folded into its prologue
//   2. rotary + K/V scatter into the paged pool
//   3. paged attention (+ split merge when the KV axis is split)
//   4. o projection with the residual add as its epilogue
//   5. interleaved [gate;up] projection, RMSNorm prologue, SwiGLU epilogue
//   6. down projection with the residual add as its epilogue
// and the LM head takes the final RMSNorm as its prologue.  Every K/V write of a
// layer precedes that layer's attention in stream order, which is what makes
// several positions of one sequence in one batch causal (src/model.rs:960-966).
#include <math.h>
#include <string.h>

#include <algorithm>
#include <new>

#include "pi_common.cuh"

struct pi_model {
  pi_model_config cfg;
  int hd = 0, heads_local = 0, kv_heads_local = 0, inter_local = 0, vocab_local = 0;
  uint16_t* embed = nullptr;
  float* final_norm = nullptr;
  std::vector<float*> attn_norm, ffn_norm;
  std::vector<pi_linear*> qkv, wo, gate_up, down;
  pi_linear* lm_head = nullptr;
  float *rope_cos = nullptr, *rope_sin = nullptr;
  int rope_cap = 0;
  // scratch for `capacity` batch rows
  int capacity = 0;
  float *x = nullptr, *qkv_buf = nullptr, *attn_out = nullptr, *h = nullptr, *partial = nullptr, *logits = nullptr,
        *logits_gather = nullptr;
  uint32_t* tokens_dev = nullptr;
  uint32_t* argmax_dev = nullptr;
  // activations handed from one tensor-core projection to the next as bf16 planes (tp == 1): the residual stream
  // (times the next norm weight) and the SwiGLU output, plus the per-tile sums of squares of the residual rows
  __nv_bfloat16 *planes_x = nullptr, *planes_h = nullptr, *planes_a = nullptr;
  float* sumsq = nullptr;
  int sumsq_tiles_cap = 0;
  size_t weight_bytes = 0;
  // pi_model_decode_multi: the executable graph of one decode step, kept between calls.  Every call captures its step
  // anew (the launch parameters depend on the batch) and updates this executable in place, which is much cheaper than
  // instantiating one; only a change of topology (another batch shape, another kernel choice) rebuilds it.
  cudaGraphExec_t step_exec = nullptr;
};

namespace {

size_t esize(int kind) { return kind == PI_INT8 ? 1 : kind == PI_BF16 ? 2 : 4; }

struct Source {
  const pi_tensor* host = nullptr;  // host tensor, or
  bool synthetic = false;           // device-generated N(0, std)
  uint64_t seed = 0, stream_id = 0;
  float std = 0.02f;
  int kind = PI_F32;                // synthetic: kind AFTER load (PI_INT8 or PI_BF16)
  size_t rows = 0, cols = 0;
};

// Load rows [src_r0, src_r0 + nrows) x cols [c0, c0 + dst->cols) of a source into
// dst rows dst_r0, dst_r0 + step, ...  Whole rows are quantised before the
// column slice is taken, so shards carry whole-row scales.
pi_status load_rows(pi_ctx* ctx, pi_linear* dst, size_t dst_r0, size_t step, const Source& s, size_t src_r0,
                    size_t nrows, size_t c0) {
  const size_t cols = s.cols;
  const int dkind = dst->kind;
  const size_t des = esize(dkind);
  const size_t chunk_rows = std::max<size_t>(1, std::min<size_t>(nrows, ((size_t)48 << 20) / cols));
  for (size_t done = 0; done < nrows; done += chunk_rows) {
    const size_t nr = std::min(chunk_rows, nrows - done);
    const size_t r0 = src_r0 + done;
    char* drow = static_cast<char*>(dst->w) + (dst_r0 + done * step) * dst->ld * des;
    float* dsc = dst->scales ? dst->scales + dst_r0 + done * step : nullptr;
    const size_t dpitch = dst->ld * des * step;

    int skind = s.synthetic ? PI_F32 : s.host->kind;
    const bool quantize = s.synthetic ? (s.kind == PI_INT8) : (s.host->quantize_on_load != 0 && skind != PI_INT8);
    const void* src_dev = nullptr;  // [nr][cols] of skind on the device
    if (s.synthetic) {
      PI_TRY(pi_reserve(ctx, &ctx->staging_in, nr * cols * sizeof(float)));
      // element index within the full matrix keeps shards consistent with the whole
      PI_REQUIRE(ctx, (r0 * cols) % 2 == 0, "synthetic rows must start on an even element");
      PI_TRY(pi_launch_fill_normal(ctx, static_cast<float*>(ctx->staging_in.ptr), nr * cols, s.seed,
                                   s.stream_id, (r0 * cols) / 2, s.std));
      src_dev = ctx->staging_in.ptr;
    } else if (skind == PI_INT8 || (!quantize && skind == dkind)) {
      // straight 2-D copy from the host
      const char* hp = static_cast<const char*>(s.host->data) + (r0 * cols + c0) * esize(skind);
      PI_REQUIRE(ctx, skind == dkind, "projection kinds of a fused matrix differ");
      PI_CUDA(ctx, cudaMemcpy2DAsync(drow, dpitch, hp, cols * des, dst->cols * des, nr, cudaMemcpyHostToDevice, ctx->stream));
      if (skind == PI_INT8)
        PI_CUDA(ctx, cudaMemcpy2DAsync(dsc, sizeof(float) * step, s.host->scales + r0, sizeof(float), sizeof(float), nr,
                                       cudaMemcpyHostToDevice, ctx->stream));
      PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      continue;
    } else {
      const size_t bytes = nr * cols * esize(skind);
      PI_TRY(pi_reserve(ctx, &ctx->staging_in, nr * cols * sizeof(float) + bytes + 256));
      char* raw = static_cast<char*>(ctx->staging_in.ptr) + nr * cols * sizeof(float);
      raw = reinterpret_cast<char*>(((uintptr_t)raw + 255) & ~(uintptr_t)255);
      const char* hp = static_cast<const char*>(s.host->data) + r0 * cols * esize(skind);
      if (skind == PI_F32) {
        PI_CUDA(ctx, cudaMemcpyAsync(ctx->staging_in.ptr, hp, bytes, cudaMemcpyHostToDevice, ctx->stream));
      } else {
        PI_CUDA(ctx, cudaMemcpyAsync(raw, hp, bytes, cudaMemcpyHostToDevice, ctx->stream));
        PI_TRY(pi_launch_bf16_to_f32(ctx, reinterpret_cast<const uint16_t*>(raw), cols,
                                     static_cast<float*>(ctx->staging_in.ptr), cols, nr, cols));
      }
      src_dev = ctx->staging_in.ptr;
      skind = PI_F32;
    }
    // src_dev holds f32 rows here
    if (quantize) {
      PI_REQUIRE(ctx, dkind == PI_INT8, "projection kinds of a fused matrix differ");
      PI_TRY(pi_reserve(ctx, &ctx->staging_out, nr * cols + nr * sizeof(float) + 16));
      float* sc = static_cast<float*>(ctx->staging_out.ptr);
      int8_t* q = reinterpret_cast<int8_t*>(sc + nr);
      PI_TRY(pi_launch_quantize(ctx, static_cast<const float*>(src_dev), cols, nr, cols, q, cols, sc));
      PI_CUDA(ctx, cudaMemcpy2DAsync(drow, dpitch, q + c0, cols, dst->cols, nr, cudaMemcpyDeviceToDevice, ctx->stream));
      PI_CUDA(ctx, cudaMemcpy2DAsync(dsc, sizeof(float) * step, sc, sizeof(float), sizeof(float), nr,
                                     cudaMemcpyDeviceToDevice, ctx->stream));
    } else if (dkind == PI_BF16) {
      PI_TRY(pi_reserve(ctx, &ctx->staging_out, nr * cols * sizeof(uint16_t)));
      PI_TRY(pi_launch_f32_to_bf16(ctx, static_cast<const float*>(src_dev), static_cast<uint16_t*>(ctx->staging_out.ptr), nr * cols));
      PI_CUDA(ctx, cudaMemcpy2DAsync(drow, dpitch, static_cast<uint16_t*>(ctx->staging_out.ptr) + c0, cols * 2,
                                     dst->cols * 2, nr, cudaMemcpyDeviceToDevice, ctx->stream));
    } else {
      PI_REQUIRE(ctx, dkind == PI_F32, "projection kinds of a fused matrix differ");
      PI_CUDA(ctx, cudaMemcpy2DAsync(drow, dpitch, static_cast<const float*>(src_dev) + c0, cols * 4, dst->cols * 4, nr,
                                     cudaMemcpyDeviceToDevice, ctx->stream));
    }
    PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  return PI_OK;
}

int loaded_kind(const Source& s) {
  if (s.synthetic) return s.kind;
  if (s.host->kind == PI_INT8 || s.host->quantize_on_load) return PI_INT8;
  return s.host->kind;
}

// A local (per-rank) matrix whose rows are slices of one or more sources.
struct Piece {
  Source src;
  size_t src_r0, nrows;  // rows taken from the source
  size_t dst_r0, step;   // where they land
};

pi_status build_linear(pi_ctx* ctx, const std::vector<Piece>& pieces, size_t local_rows, size_t local_cols, size_t c0,
                       pi_linear** out) {
  const int kind = loaded_kind(pieces[0].src);
  for (const Piece& p : pieces) PI_REQUIRE(ctx, loaded_kind(p.src) == kind, "projections fused into one matrix must share a kind");
  // Allocate as an unsharded matrix of the local shape; sharding is done by the pieces.
  const int tp = ctx->tp;
  ctx->tp = 1;
  pi_status s = pi_linear_alloc(ctx, kind, local_rows, local_cols, PI_SPLIT_NONE, out);
  ctx->tp = tp;
  PI_TRY(s);
  pi_linear* lin = *out;
  if (lin->ld != lin->cols) PI_CUDA(ctx, cudaMemsetAsync(lin->w, 0, lin->rows * lin->ld * esize(kind), ctx->stream));
  for (const Piece& p : pieces) PI_TRY(load_rows(ctx, lin, p.dst_r0, p.step, p.src, p.src_r0, p.nrows, c0));
  return PI_OK;
}

pi_status alloc_f(pi_ctx* ctx, float** p, size_t n) {
  PI_CUDA(ctx, cudaMalloc(p, std::max<size_t>(n, 1) * sizeof(float)));
  return PI_OK;
}

pi_status ensure_rope(pi_ctx* ctx, pi_model* m, int positions) {
  if (positions <= m->rope_cap) return PI_OK;
  int cap = std::max(positions, std::max(m->rope_cap * 2, 256));
  const int half = m->hd / 2;
  std::vector<float> c((size_t)cap * std::max(half, 1)), s((size_t)cap * std::max(half, 1));
  for (int p = 0; p < cap; ++p) pi_host_rope_table(p, m->hd, m->cfg.rope_theta, &c[(size_t)p * half], &s[(size_t)p * half]);
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (m->rope_cos) cudaFree(m->rope_cos);
  if (m->rope_sin) cudaFree(m->rope_sin);
  m->rope_cos = m->rope_sin = nullptr;
  PI_TRY(alloc_f(ctx, &m->rope_cos, c.size()));
  PI_TRY(alloc_f(ctx, &m->rope_sin, s.size()));
  PI_CUDA(ctx, cudaMemcpy(m->rope_cos, c.data(), c.size() * sizeof(float), cudaMemcpyHostToDevice));
  PI_CUDA(ctx, cudaMemcpy(m->rope_sin, s.data(), s.size() * sizeof(float), cudaMemcpyHostToDevice));
  m->rope_cap = cap;
  return PI_OK;
}

pi_status validate_config(pi_ctx* ctx, const pi_model_config* c) {
  PI_REQUIRE(ctx, c->hidden_size > 0 && c->num_hidden_layers > 0 && c->num_attention_heads > 0 &&
                      c->num_key_value_heads > 0 && c->intermediate_size > 0 && c->vocab_size > 0,
             "model config fields must be positive");
  PI_REQUIRE(ctx, c->hidden_size % c->num_attention_heads == 0, "hidden_size must be a multiple of num_attention_heads");
  PI_REQUIRE(ctx, c->num_attention_heads % c->num_key_value_heads == 0,
             "num_attention_heads (%d) must be a multiple of num_key_value_heads (%d)", c->num_attention_heads,
             c->num_key_value_heads);
  PI_REQUIRE(ctx, c->rope_style == 0 || c->rope_style == 1, "rope_style must be 0 or 1");
  PI_REQUIRE(ctx, c->max_batch > 0, "max_batch must be positive");
  if (ctx->tp > 1) {
    PI_REQUIRE(ctx, c->num_key_value_heads % ctx->tp == 0, "%d KV heads do not split over %d ranks", c->num_key_value_heads, ctx->tp);
    PI_REQUIRE(ctx, c->intermediate_size % ctx->tp == 0 && c->vocab_size % ctx->tp == 0,
               "intermediate_size and vocab_size must be multiples of the tensor-parallel degree");
  }
  return PI_OK;
}

// Sources for the seven projections of a layer + lm_head.
struct ModelSources {
  std::vector<Source> proj;  // [layers*7]
  Source lm_head;
};

pi_status build_model(pi_ctx* ctx, const pi_model_config* cfg, const ModelSources& src, const uint16_t* embed_host,
                      const float* final_norm_host, const float* const* attn_norm_host,
                      const float* const* ffn_norm_host, uint64_t synth_seed, pi_model* m) {
  m->cfg = *cfg;
  const int tp = ctx->tp, rank = ctx->rank;
  const int H = cfg->num_attention_heads, KH = cfg->num_key_value_heads, hidden = cfg->hidden_size;
  const int hd = hidden / H, inter = cfg->intermediate_size, vocab = cfg->vocab_size, NL = cfg->num_hidden_layers;
  m->hd = hd;
  m->heads_local = H / tp;
  m->kv_heads_local = KH / tp;
  m->inter_local = inter / tp;
  m->vocab_local = vocab / tp;
  const size_t qrows = (size_t)m->heads_local * hd, kvrows = (size_t)m->kv_heads_local * hd;

  // embeddings + norms (replicated)
  PI_CUDA(ctx, cudaMalloc(&m->embed, (size_t)vocab * hidden * sizeof(uint16_t)));
  PI_TRY(alloc_f(ctx, &m->final_norm, hidden));
  if (embed_host) {
    PI_CUDA(ctx, cudaMemcpy(m->embed, embed_host, (size_t)vocab * hidden * sizeof(uint16_t), cudaMemcpyHostToDevice));
    PI_CUDA(ctx, cudaMemcpy(m->final_norm, final_norm_host, hidden * sizeof(float), cudaMemcpyHostToDevice));
  } else {
    const size_t n = (size_t)vocab * hidden;
    PI_TRY(pi_reserve(ctx, &ctx->staging_in, n * sizeof(float)));
    PI_TRY(pi_launch_fill_normal(ctx, static_cast<float*>(ctx->staging_in.ptr), n, synth_seed, 0xE0000000ull, 0, 0.02f));
    PI_TRY(pi_launch_f32_to_bf16(ctx, static_cast<float*>(ctx->staging_in.ptr), m->embed, n));
    std::vector<float> ones(hidden, 1.0f);
    PI_CUDA(ctx, cudaMemcpyAsync(m->final_norm, ones.data(), hidden * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  m->attn_norm.assign(NL, nullptr);
  m->ffn_norm.assign(NL, nullptr);
  std::vector<float> ones(hidden, 1.0f);
  for (int l = 0; l < NL; ++l) {
    PI_TRY(alloc_f(ctx, &m->attn_norm[l], hidden));
    PI_TRY(alloc_f(ctx, &m->ffn_norm[l], hidden));
    PI_CUDA(ctx, cudaMemcpy(m->attn_norm[l], attn_norm_host ? attn_norm_host[l] : ones.data(), hidden * sizeof(float), cudaMemcpyHostToDevice));
    PI_CUDA(ctx, cudaMemcpy(m->ffn_norm[l], ffn_norm_host ? ffn_norm_host[l] : ones.data(), hidden * sizeof(float), cudaMemcpyHostToDevice));
  }

  m->qkv.assign(NL, nullptr);
  m->wo.assign(NL, nullptr);
  m->gate_up.assign(NL, nullptr);
  m->down.assign(NL, nullptr);
  for (int l = 0; l < NL; ++l) {
    const Source* p = &src.proj[(size_t)l * 7];
    PI_REQUIRE(ctx, p[0].rows == (size_t)hidden && p[0].cols == (size_t)hidden, "layer %d wq must be %dx%d", l, hidden, hidden);
    PI_REQUIRE(ctx, p[1].rows == (size_t)KH * hd && p[1].cols == (size_t)hidden, "layer %d wk has the wrong shape", l);
    PI_REQUIRE(ctx, p[2].rows == (size_t)KH * hd && p[2].cols == (size_t)hidden, "layer %d wv has the wrong shape", l);
    PI_REQUIRE(ctx, p[3].rows == (size_t)hidden && p[3].cols == (size_t)hidden, "layer %d wo has the wrong shape", l);
    PI_REQUIRE(ctx, p[4].rows == (size_t)inter && p[4].cols == (size_t)hidden, "layer %d w1 has the wrong shape", l);
    PI_REQUIRE(ctx, p[5].rows == (size_t)hidden && p[5].cols == (size_t)inter, "layer %d w2 has the wrong shape", l);
    PI_REQUIRE(ctx, p[6].rows == (size_t)inter && p[6].cols == (size_t)hidden, "layer %d w3 has the wrong shape", l);
    // column split: this rank's heads / FFN rows.  row split: this rank's input columns.
    PI_TRY(build_linear(ctx, {{p[0], rank * qrows, qrows, 0, 1}, {p[1], rank * kvrows, kvrows, qrows, 1},
                              {p[2], rank * kvrows, kvrows, qrows + kvrows, 1}},
                        qrows + 2 * kvrows, hidden, 0, &m->qkv[l]));
    PI_TRY(build_linear(ctx, {{p[3], 0, (size_t)hidden, 0, 1}}, hidden, qrows, rank * qrows, &m->wo[l]));
    const size_t il = m->inter_local;
    PI_TRY(build_linear(ctx, {{p[4], rank * il, il, 0, 2}, {p[6], rank * il, il, 1, 2}}, 2 * il, hidden, 0, &m->gate_up[l]));
    PI_TRY(build_linear(ctx, {{p[5], 0, (size_t)hidden, 0, 1}}, hidden, il, rank * il, &m->down[l]));
    for (pi_linear* lin : {m->qkv[l], m->wo[l], m->gate_up[l], m->down[l]}) m->weight_bytes += pi_linear_weight_bytes(lin);
  }
  PI_REQUIRE(ctx, src.lm_head.rows == (size_t)vocab && src.lm_head.cols == (size_t)hidden, "lm_head has the wrong shape");
  PI_TRY(build_linear(ctx, {{src.lm_head, (size_t)rank * m->vocab_local, (size_t)m->vocab_local, 0, 1}}, m->vocab_local,
                      hidden, 0, &m->lm_head));
  m->weight_bytes += pi_linear_weight_bytes(m->lm_head);

  // scratch
  const size_t cap = cfg->max_batch;
  m->capacity = cfg->max_batch;
  PI_TRY(alloc_f(ctx, &m->x, cap * hidden));
  PI_TRY(alloc_f(ctx, &m->qkv_buf, cap * (qrows + 2 * kvrows)));
  PI_TRY(alloc_f(ctx, &m->attn_out, cap * qrows));
  PI_TRY(alloc_f(ctx, &m->h, cap * m->inter_local));
  PI_TRY(alloc_f(ctx, &m->partial, cap * hidden));
  PI_TRY(alloc_f(ctx, &m->logits, cap * vocab));
  if (tp > 1) PI_TRY(alloc_f(ctx, &m->logits_gather, cap * vocab));
  PI_CUDA(ctx, cudaMalloc(&m->tokens_dev, cap * sizeof(uint32_t)));
  PI_CUDA(ctx, cudaMalloc(&m->argmax_dev, cap * sizeof(uint32_t)));
  {
    PI_CUDA(ctx, cudaMalloc(&m->planes_x, 3 * cap * hidden * sizeof(__nv_bfloat16)));
    PI_CUDA(ctx, cudaMalloc(&m->planes_h, 3 * cap * (size_t)m->inter_local * sizeof(__nv_bfloat16)));
    PI_CUDA(ctx, cudaMalloc(&m->planes_a, 3 * cap * qrows * sizeof(__nv_bfloat16)));
    m->sumsq_tiles_cap = (hidden + 127) / 128;
    PI_TRY(alloc_f(ctx, &m->sumsq, (size_t)m->sumsq_tiles_cap * cap));
  }
  PI_TRY(ensure_rope(ctx, m, cfg->max_positions > 0 ? cfg->max_positions : 4096));
  PI_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return PI_OK;
}

// [tp][B][V/tp] -> [B][V]
__global__ void gather_logits_kernel(const float* __restrict__ in, float* __restrict__ out, int tp, int B, int vl) {
  const size_t total = (size_t)tp * B * vl;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vl);
    const size_t t = i / vl;
    const int b = (int)(t % B), r = (int)(t / B);
    out[((size_t)b * tp + r) * vl + v] = in[i];
  }
}

// What the last projection of run_layers left for the LM head when it could emit planes (tp == 1, tensor path).
struct x_planes_state {
  pi_act_planes planes;
  bool valid = false;
};

// run_layers_batch: leaves the residual stream (before the final norm) in m->x.  On the tensor-core path with
// tp == 1 the projections pass their result on as bf16 planes (already multiplied by the next norm weight, with the
// sums of squares the next projection turns into 1/rms): o -> gate/up -> down -> next layer's q/k/v (or the LM
// head, through `final_x`), so only the attention output and the embeddings go through the split kernel.
pi_status run_layers(pi_ctx* ctx, pi_model* m, pi_kv_pool* pool, const pi_attn_batch& batch, int B, x_planes_state* final_x) {
  const pi_model_config& c = m->cfg;
  const int hidden = c.hidden_size, hd = m->hd, L = c.num_hidden_layers;
  const size_t qrows = (size_t)m->heads_local * hd, kvrows = (size_t)m->kv_heads_local * hd;
  const size_t qkv_stride = qrows + 2 * kvrows;
  const size_t cap = (size_t)m->capacity;
  const bool peer = pi_tp_peer_usable(ctx, (size_t)B * hidden);   // partial sums exchanged through peer memory
  const bool fuse = ctx->opt_fuse_planes && (ctx->tp == 1 || peer) && m->planes_x && m->planes_h;
  pi_act_planes px, ph, pa;            // residual-stream planes, SwiGLU-output planes, attention-output planes
  px.base = m->planes_x; px.plane_stride = cap * hidden; px.K = hidden;
  px.sumsq = m->sumsq; px.sumsq_stride = cap;
  ph.base = m->planes_h; ph.plane_stride = cap * (size_t)m->inter_local; ph.K = m->inter_local;
  pa.base = m->planes_a; pa.plane_stride = cap * qrows; pa.K = (int)qrows;
  bool x_ready = false;                // px holds the planes of m->x for the next norm
  if (final_x) final_x->valid = false;

  PI_TRY(pi_attention_prepare(ctx, pool, m->heads_local, batch));   // the step's work list, from the positions on the device
  PI_TRY(pi_launch_embed(ctx, m->embed, c.vocab_size, hidden, m->tokens_dev, B, m->x));
  for (int l = 0; l < L; ++l) {
    pi_linear_args a;
    a.M = B;
    a.x = m->x;
    a.x_stride = hidden;
    a.out = m->qkv_buf;
    a.out_stride = qkv_stride;
    a.norm_weight = m->attn_norm[l];
    a.norm_eps = c.rms_norm_eps;
    if (x_ready) a.in_planes = &px;
    pi_rope_kv rk;
    rk.num_heads = m->heads_local;
    rk.num_kv_heads = m->kv_heads_local;
    rk.head_dim = hd;
    rk.style = c.rope_style;
    rk.rope_cos = m->rope_cos;
    rk.rope_sin = m->rope_sin;
    rk.pool = pool;
    rk.layer = l;
    rk.batch = &batch;
    const bool rope_fused = ctx->opt_fuse_planes && (pi_gemm_tc_will_run(ctx, m->qkv[l], a) ? pi_gemm_tc_can_rope(ctx, m->qkv[l], a, rk)
                                                                                             : pi_gemv_can_rope(ctx, m->qkv[l], a, rk));
    if (rope_fused) a.rope = &rk;
    PI_TRY(pi_linear_forward(ctx, m->qkv[l], a));
    x_ready = false;
    if (!rope_fused)
      PI_TRY(pi_launch_rope_kv_write(ctx, m->qkv_buf, qkv_stride, m->heads_local, m->kv_heads_local, hd, m->rope_cos,
                                     m->rope_sin, c.rope_style, pool, l, batch));
    pi_linear_args o;
    o.M = B;
    o.x = m->attn_out;
    o.x_stride = qrows;
    bool a_ready = false;              // the merge kernel of the attention wrote the output as planes too
    const bool o_tc = fuse && m->planes_a && pi_gemm_tc_will_run(ctx, m->wo[l], o);
    batch.flat_settled = l > 0;   // the work list of the step was complete long before the kernel ahead of this launch started
    PI_TRY(pi_launch_attention(ctx, pool, l, m->heads_local, m->qkv_buf, qkv_stride, m->attn_out, qrows, batch,
                               o_tc ? &pa : nullptr, &a_ready));
    if (a_ready) o.in_planes = &pa;

    // gate/up consumes planes only if it runs on the tensor path itself
    pi_linear_args g;
    g.M = B;
    g.x = m->x;
    g.x_stride = hidden;
    g.out = m->h;
    g.out_stride = m->inter_local;
    g.norm_weight = m->ffn_norm[l];
    g.norm_eps = c.rms_norm_eps;
    g.epi = PI_EPI_SWIGLU;
    const bool g_tc = fuse && pi_gemm_tc_will_run(ctx, m->gate_up[l], g);

    if (ctx->tp > 1) {
      o.out = peer ? pi_tp_peer_slot(ctx) : m->partial;
      o.out_stride = hidden;
      if (peer && ctx->opt_tp_push && pi_gemm_tc_will_run(ctx, m->wo[l], o) && m->wo[l]->rows % 4 == 0)
        o.n_out_also = pi_tp_peer_push_targets(ctx, o.out_also);   // the epilogue stores into the peers' buffers too
      PI_TRY(pi_linear_forward(ctx, m->wo[l], o));
      if (peer) {   // the exchange kernel adds the residual and hands the new rows on as planes
        x_ready = g_tc;
        PI_TRY(pi_tp_peer_reduce_add(ctx, m->x, B, hidden, x_ready ? &px : nullptr, m->ffn_norm[l], c.rms_norm_eps));
      } else {
        PI_TRY(pi_tp_all_reduce_sum(ctx, m->partial, (size_t)B * hidden));
        PI_TRY(pi_launch_add(ctx, m->x, m->partial, (size_t)B * hidden));
      }
    } else {
      o.out = m->x;
      o.out_stride = hidden;
      o.epi = PI_EPI_ADD;
      if (g_tc && pi_gemm_tc_can_emit(ctx, m->wo[l], o, true)) {
        o.emit = &px;
        o.emit_norm_weight = m->ffn_norm[l];
        o.emit_norm_eps = c.rms_norm_eps;
        x_ready = true;
      }
      PI_TRY(pi_linear_forward(ctx, m->wo[l], o));
    }

    pi_linear_args d;
    d.M = B;
    d.x = m->h;
    d.x_stride = m->inter_local;
    const bool d_tc = fuse && pi_gemm_tc_will_run(ctx, m->down[l], d);
    bool h_ready = false;
    if (x_ready) g.in_planes = &px;
    if (d_tc && pi_gemm_tc_can_emit(ctx, m->gate_up[l], g, false)) {
      g.emit = &ph;
      h_ready = true;
    }
    PI_TRY(pi_linear_forward(ctx, m->gate_up[l], g));
    x_ready = false;

    if (ctx->tp > 1) {
      d.out = peer ? pi_tp_peer_slot(ctx) : m->partial;
      d.out_stride = hidden;
      if (h_ready) d.in_planes = &ph;
      if (peer && ctx->opt_tp_push && pi_gemm_tc_will_run(ctx, m->down[l], d) && m->down[l]->rows % 4 == 0)
        d.n_out_also = pi_tp_peer_push_targets(ctx, d.out_also);
      PI_TRY(pi_linear_forward(ctx, m->down[l], d));
      if (peer) {
        const pi_linear* next = l + 1 < L ? m->qkv[l + 1] : (final_x ? m->lm_head : nullptr);
        pi_linear_args nx;
        nx.M = B;
        x_ready = fuse && next && pi_gemm_tc_will_run(ctx, next, nx);
        PI_TRY(pi_tp_peer_reduce_add(ctx, m->x, B, hidden, x_ready ? &px : nullptr,
                                     l + 1 < L ? m->attn_norm[l + 1] : m->final_norm, c.rms_norm_eps));
      } else {
        PI_TRY(pi_tp_all_reduce_sum(ctx, m->partial, (size_t)B * hidden));
        PI_TRY(pi_launch_add(ctx, m->x, m->partial, (size_t)B * hidden));
      }
    } else {
      d.out = m->x;
      d.out_stride = hidden;
      d.epi = PI_EPI_ADD;
      if (h_ready) d.in_planes = &ph;
      // the consumer of the new residual stream: the next layer's q/k/v, or the LM head over all B rows
      const pi_linear* next = l + 1 < L ? m->qkv[l + 1] : (final_x ? m->lm_head : nullptr);
      pi_linear_args nx;
      nx.M = B;
      if (fuse && next && pi_gemm_tc_will_run(ctx, next, nx) && pi_gemm_tc_can_emit(ctx, m->down[l], d, true)) {
        d.emit = &px;
        d.emit_norm_weight = l + 1 < L ? m->attn_norm[l + 1] : m->final_norm;
        d.emit_norm_eps = c.rms_norm_eps;
        x_ready = true;
      }
      PI_TRY(pi_linear_forward(ctx, m->down[l], d));
    }
  }
  if (final_x && x_ready) {
    final_x->planes = px;
    final_x->valid = true;
  }
  return PI_OK;
}

// Final norm + LM head for `rows` rows of m->x starting at row `first`; logits land in m->logits [rows][vocab].
// `xp`: planes of all rows of m->x times the final norm weight, when run_layers left them (first must be 0).
pi_status project_logits(pi_ctx* ctx, pi_model* m, int first, int rows, const x_planes_state* xp = nullptr) {
  const pi_model_config& c = m->cfg;
  pi_linear_args a;
  a.M = rows;
  a.x = m->x + (size_t)first * c.hidden_size;
  a.x_stride = c.hidden_size;
  a.norm_weight = m->final_norm;
  a.norm_eps = c.rms_norm_eps;
  if (ctx->tp > 1) {
    a.out = m->logits;  // [rows][vocab_local]
    a.out_stride = m->vocab_local;
    if (xp && xp->valid && first == 0) a.in_planes = &xp->planes;
    PI_TRY(pi_linear_forward(ctx, m->lm_head, a));
    PI_TRY(pi_tp_all_gather(ctx, m->logits, m->logits_gather, (size_t)rows * m->vocab_local * sizeof(float)));
    const size_t total = (size_t)rows * c.vocab_size;
    gather_logits_kernel<<<(unsigned)std::min<size_t>((total + 255) / 256, 4096), 256, 0, ctx->stream>>>(
        m->logits_gather, m->logits, ctx->tp, rows, m->vocab_local);
    PI_CHECK_LAUNCH(ctx);
  } else {
    a.out = m->logits;
    a.out_stride = c.vocab_size;
    if (xp && xp->valid && first == 0) a.in_planes = &xp->planes;
    PI_TRY(pi_linear_forward(ctx, m->lm_head, a));
  }
  return PI_OK;
}

pi_status fetch_results(pi_ctx* ctx, pi_model* m, int rows, float* logits_host, uint32_t* argmax_host) {
  const int vocab = m->cfg.vocab_size;
  if (argmax_host) {
    PI_TRY(pi_launch_argmax(ctx, m->logits, vocab, rows, vocab, m->argmax_dev));
    PI_CUDA(ctx, cudaMemcpyAsync(argmax_host, m->argmax_dev, rows * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  }
  if (logits_host)
    PI_CUDA(ctx, cudaMemcpyAsync(logits_host, m->logits, (size_t)rows * vocab * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  return PI_OK;
}

pi_status check_pool(pi_ctx* ctx, const pi_model* m, const pi_kv_pool* pool) {
  PI_REQUIRE(ctx, pool != nullptr, "null KV pool");
  PI_REQUIRE(ctx, pool->L.num_layers == m->cfg.num_hidden_layers && pool->L.num_kv_heads == m->kv_heads_local &&
                      pool->L.head_dim == m->hd,
             "KV pool layout (%d layers, %d kv heads, head_dim %d) does not match the model (%d, %d, %d)",
             pool->L.num_layers, pool->L.num_kv_heads, pool->L.head_dim, m->cfg.num_hidden_layers, m->kv_heads_local, m->hd);
  return PI_OK;
}

// Upload one batch: tokens, tables, positions; window starts from the config.
pi_status stage_batch(pi_ctx* ctx, pi_model* m, pi_kv_pool* pool, const uint32_t* tokens, const int32_t* positions,
                      const int32_t* tables, int max_blocks, const int32_t* lens, int B, pi_attn_batch* batch) {
  std::vector<int32_t> start(B);
  int max_pos = 0;
  for (int b = 0; b < B; ++b) {
    PI_REQUIRE(ctx, positions[b] >= 0, "entry %d: negative position", b);
    const int w = m->cfg.attention_window;
    start[b] = w < 0 ? 0 : std::max(0, positions[b] + 1 - w);  // AttnEntry::new
    max_pos = std::max(max_pos, positions[b]);
    for (int i = 0; i < lens[b] && i < max_blocks; ++i) {
      const int32_t pb = tables[(size_t)b * max_blocks + i];
      PI_REQUIRE(ctx, pb >= 0 && pb < pool->L.num_blocks, "entry %d maps a block to physical id %d of %d", b, pb, pool->L.num_blocks);
    }
  }
  PI_TRY(ensure_rope(ctx, m, max_pos + 1));
  PI_TRY(pi_upload_attn_batch(ctx, tables, max_blocks, lens, positions, start.data(), B, pool->L.block_size, pool->L.num_blocks, batch));
  PI_CUDA(ctx, cudaMemcpyAsync(m->tokens_dev, tokens, B * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream));
  return PI_OK;
}

}  // namespace

extern "C" {

pi_status pi_model_create(pi_ctx* ctx, const pi_model_config* cfg, const pi_model_weights* w, pi_model** out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, cfg && w && out, "null pointer");
  *out = nullptr;
  PI_TRY(validate_config(ctx, cfg));
  PI_REQUIRE(ctx, w->token_embeddings_bf16 && w->final_norm && w->attention_norm && w->ffn_norm && w->projections, "null weight pointer");
  ModelSources src;
  src.proj.resize((size_t)cfg->num_hidden_layers * 7);
  auto mk = [&](const pi_tensor& t, Source* s) -> pi_status {
    PI_REQUIRE(ctx, t.data != nullptr, "null projection data");
    PI_REQUIRE(ctx, t.kind == PI_F32 || t.kind == PI_INT8 || t.kind == PI_BF16, "unknown weight kind %d", t.kind);
    PI_REQUIRE(ctx, t.kind != PI_INT8 || t.scales != nullptr, "int8 projection without scales");
    s->host = &t;
    s->rows = (size_t)t.rows;
    s->cols = (size_t)t.cols;
    return PI_OK;
  };
  for (size_t i = 0; i < src.proj.size(); ++i) PI_TRY(mk(w->projections[i], &src.proj[i]));
  PI_TRY(mk(w->lm_head, &src.lm_head));
  pi_model* m = new (std::nothrow) pi_model();
  if (!m) return pi_fail(ctx, PI_ERR_OOM, "host allocation failed");
  pi_status s = build_model(ctx, cfg, src, w->token_embeddings_bf16, w->final_norm, w->attention_norm, w->ffn_norm, 0, m);
  if (s != PI_OK) {
    pi_model_destroy(m);
    return s;
  }
  *out = m;
  return PI_OK;
}

pi_status pi_model_create_synthetic(pi_ctx* ctx, const pi_model_config* cfg, uint64_t seed, float std, int quant,
                                    int lm_head_kind, pi_model** out) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, cfg && out, "null pointer");
  *out = nullptr;
  PI_TRY(validate_config(ctx, cfg));
  PI_REQUIRE(ctx, (quant == PI_INT8 || quant == PI_BF16) && (lm_head_kind == PI_INT8 || lm_head_kind == PI_BF16),
             "synthetic weights are int8 or bf16");
  const size_t hidden = cfg->hidden_size, inter = cfg->intermediate_size;
  const size_t kvd = (size_t)cfg->num_key_value_heads * (hidden / cfg->num_attention_heads);
  PI_REQUIRE(ctx, hidden % 2 == 0 && inter % 2 == 0, "synthetic weights need even dimensions");
  const size_t shapes[7][2] = {{hidden, hidden}, {kvd, hidden}, {kvd, hidden}, {hidden, hidden},
                               {inter, hidden},  {hidden, inter}, {inter, hidden}};
  ModelSources src;
  src.proj.resize((size_t)cfg->num_hidden_layers * 7);
  for (size_t i = 0; i < src.proj.size(); ++i) {
    Source& s = src.proj[i];
    s.synthetic = true;
    s.seed = seed;
    s.stream_id = i + 1;
    s.std = std;
    s.kind = quant;
    s.rows = shapes[i % 7][0];
    s.cols = shapes[i % 7][1];
  }
  src.lm_head.synthetic = true;
  src.lm_head.seed = seed;
  src.lm_head.stream_id = 0xF0000000ull;
  src.lm_head.std = std;
  src.lm_head.kind = lm_head_kind;
  src.lm_head.rows = cfg->vocab_size;
  src.lm_head.cols = hidden;
  pi_model* m = new (std::nothrow) pi_model();
  if (!m) return pi_fail(ctx, PI_ERR_OOM, "host allocation failed");
  pi_status s = build_model(ctx, cfg, src, nullptr, nullptr, nullptr, nullptr, seed, m);
  if (s != PI_OK) {
    pi_model_destroy(m);
    return s;
  }
  *out = m;
  return PI_OK;
}

void pi_model_destroy(pi_model* m) {
  if (!m) return;
  if (m->step_exec) cudaGraphExecDestroy(m->step_exec);
  for (auto* v : {&m->qkv, &m->wo, &m->gate_up, &m->down})
    for (pi_linear* l : *v) pi_linear_destroy(l);
  pi_linear_destroy(m->lm_head);
  for (float* p : m->attn_norm) cudaFree(p);
  for (float* p : m->ffn_norm) cudaFree(p);
  for (void* p : {(void*)m->embed, (void*)m->final_norm, (void*)m->rope_cos, (void*)m->rope_sin, (void*)m->x,
                  (void*)m->qkv_buf, (void*)m->attn_out, (void*)m->h, (void*)m->partial, (void*)m->logits,
                  (void*)m->logits_gather, (void*)m->tokens_dev, (void*)m->argmax_dev, (void*)m->planes_x,
                  (void*)m->planes_h, (void*)m->planes_a, (void*)m->sumsq})
    if (p) cudaFree(p);
  delete m;
}

size_t pi_model_weight_bytes(const pi_model* m) { return m ? m->weight_bytes : 0; }
int pi_model_max_batch(const pi_model* m) { return m ? m->capacity : 0; }

pi_status pi_model_decode_batch_rows(pi_ctx* ctx, pi_model* m, pi_kv_pool* pool, const uint32_t* tokens_host,
                                     const int32_t* positions_host, const int32_t* block_tables_host, int max_blocks,
                                     const int32_t* table_lens_host, int B, const int32_t* logit_rows_host, int n_logit_rows,
                                     float* logits_host, uint32_t* argmax_host) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, m && argmax_host, "null pointer");
  PI_REQUIRE(ctx, n_logit_rows >= 0 && n_logit_rows <= B && (n_logit_rows == 0 || (logit_rows_host && logits_host)),
             "%d rows of logits were asked for out of %d", n_logit_rows, B);
  for (int i = 0; i < n_logit_rows; ++i)
    PI_REQUIRE(ctx, logit_rows_host[i] >= 0 && logit_rows_host[i] < B, "logits of row %d of a batch of %d", logit_rows_host[i], B);
  // the forward and the greedy ids; the ids' copy is queued, the selected rows follow on the same stream
  PI_TRY(pi_model_decode_batch(ctx, m, pool, tokens_host, positions_host, block_tables_host, max_blocks, table_lens_host, B,
                               nullptr, nullptr));
  PI_TRY(pi_launch_argmax(ctx, m->logits, m->cfg.vocab_size, B, m->cfg.vocab_size, m->argmax_dev));
  PI_CUDA(ctx, cudaMemcpyAsync(argmax_host, m->argmax_dev, B * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  const size_t vocab = (size_t)m->cfg.vocab_size;
  for (int i = 0; i < n_logit_rows; ++i)
    PI_CUDA(ctx, cudaMemcpyAsync(logits_host + (size_t)i * vocab, m->logits + (size_t)logit_rows_host[i] * vocab,
                                 vocab * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  return pi_ctx_synchronize(ctx);
}

pi_status pi_model_decode_batch(pi_ctx* ctx, pi_model* m, pi_kv_pool* pool, const uint32_t* tokens_host,
                                const int32_t* positions_host, const int32_t* block_tables_host, int max_blocks,
                                const int32_t* table_lens_host, int B, float* logits_host_or_null,
                                uint32_t* argmax_host_or_null) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, m && tokens_host && positions_host && table_lens_host, "null pointer");
  PI_REQUIRE(ctx, block_tables_host || max_blocks == 0, "null block tables");
  PI_REQUIRE(ctx, B > 0, "decode_batch_into needs at least one sequence");
  PI_REQUIRE(ctx, B <= m->capacity, "batch %d exceeds scratch capacity %d", B, m->capacity);
  PI_TRY(check_pool(ctx, m, pool));
  pi_attn_batch batch;
  PI_TRY(stage_batch(ctx, m, pool, tokens_host, positions_host, block_tables_host, max_blocks, table_lens_host, B, &batch));
  x_planes_state xs;
  PI_TRY(run_layers(ctx, m, pool, batch, B, &xs));
  PI_TRY(project_logits(ctx, m, 0, B, &xs));
  PI_TRY(fetch_results(ctx, m, B, logits_host_or_null, argmax_host_or_null));
  if (logits_host_or_null || argmax_host_or_null) return pi_ctx_synchronize(ctx);
  return PI_OK;
}

// After a greedy step: the chosen ids become the next inputs, every sequence moves on one position.
// The step index lives on the device so that one captured graph serves every step.
static __global__ void advance_kernel(uint32_t* tokens, const uint32_t* chosen, uint32_t* history, int* step_counter,
                                      int32_t* pos, int32_t* start, int window, int B) {
  pi_grid_dependency_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  const int step = *step_counter;
  if (b < B) {
    const uint32_t t = chosen[b];
    tokens[b] = t;
    history[(size_t)step * B + b] = t;
    const int p = pos[b] + 1;
    pos[b] = p;
    start[b] = window < 0 ? 0 : max(0, p + 1 - window);
  }
  if (gridDim.x == 1) {   // a single block: it bumps the step counter itself once all its threads have read it
    __syncthreads();
    if (threadIdx.x == 0) *step_counter = step + 1;
  }
}

// Bumps the step counter once all blocks of advance_kernel are done (stream order).
static __global__ void next_step_kernel(int* step_counter) {
  pi_grid_dependency_wait();
  step_counter[0] += 1;
}

static pi_status decode_one_step(pi_ctx* ctx, pi_model* m, pi_kv_pool* pool, const pi_attn_batch& batch, int B,
                                 uint32_t* history, int* step_counter) {
  x_planes_state xs;
  PI_TRY(run_layers(ctx, m, pool, batch, B, &xs));
  PI_TRY(project_logits(ctx, m, 0, B, &xs));
  PI_TRY(pi_launch_argmax(ctx, m->logits, m->cfg.vocab_size, B, m->cfg.vocab_size, m->argmax_dev));
  pi_prof_scope prof(ctx, PI_PROF_OTHER);
  const int blocks = (B + 127) / 128;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(128);
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, advance_kernel, m->tokens_dev, (const uint32_t*)m->argmax_dev, history, step_counter,
                                           const_cast<int32_t*>(batch.pos), const_cast<int32_t*>(batch.start),
                                           m->cfg.attention_window, B);
  if (e != cudaSuccess) return pi_fail(ctx, PI_ERR_CUDA, "advance launch failed: %s", cudaGetErrorString(e));
  ctx->launches++;
  if (blocks > 1) {   // several blocks read the counter: it moves on in a launch of its own
    next_step_kernel<<<1, 1, 0, ctx->stream>>>(step_counter);
    PI_CHECK_LAUNCH(ctx);
  }
  return PI_OK;
}

pi_status pi_model_decode_multi(pi_ctx* ctx, pi_model* m, pi_kv_pool* pool, const uint32_t* tokens_host,
                                const int32_t* positions_host, const int32_t* block_tables_host, int max_blocks,
                                const int32_t* table_lens_host, int B, int n_steps, uint32_t* out_tokens_host) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, m && tokens_host && positions_host && table_lens_host && out_tokens_host, "null pointer");
  PI_REQUIRE(ctx, block_tables_host || max_blocks == 0, "null block tables");
  PI_REQUIRE(ctx, B > 0, "decode needs at least one sequence");
  PI_REQUIRE(ctx, B <= m->capacity, "batch %d exceeds scratch capacity %d", B, m->capacity);
  PI_REQUIRE(ctx, n_steps > 0, "n_steps must be positive");
  PI_TRY(check_pool(ctx, m, pool));
  int max_pos = 0;
  for (int b = 0; b < B; ++b) max_pos = std::max(max_pos, positions_host[b]);
  PI_TRY(ensure_rope(ctx, m, max_pos + n_steps));
  PI_TRY(pi_reserve(ctx, &ctx->staging_out, 64 + (size_t)n_steps * B * sizeof(uint32_t)));
  int* step_counter = static_cast<int*>(ctx->staging_out.ptr);
  uint32_t* history = reinterpret_cast<uint32_t*>(static_cast<char*>(ctx->staging_out.ptr) + 64);
  PI_CUDA(ctx, cudaMemsetAsync(step_counter, 0, 64, ctx->stream));
  pi_attn_batch batch;
  PI_TRY(stage_batch(ctx, m, pool, tokens_host, positions_host, block_tables_host, max_blocks, table_lens_host, B, &batch));
  // The KV split is planned on the host from the final positions, so that every step fits it.
  const int bs = pool->L.block_size;
  batch.total_window_blocks += (long)B * ((n_steps + bs - 1) / bs);
  batch.max_window_blocks += (n_steps + bs - 1) / bs;

  // Step 0 runs eagerly (it also sizes every scratch buffer).  The remaining steps are identical launches
  // over device-resident state, so one step is captured into a CUDA graph and replayed.
  PI_TRY(decode_one_step(ctx, m, pool, batch, B, history, step_counter));
  int done = 1;
  if (ctx->opt_graph && !ctx->prof_on && n_steps >= 4) {
    cudaGraph_t graph = nullptr;
    const uint64_t before = ctx->launches;
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
      pi_status st = decode_one_step(ctx, m, pool, batch, B, history, step_counter);
      e = cudaStreamEndCapture(ctx->stream, &graph);
      const uint64_t per_step = ctx->launches - before;
      ctx->launches = before;
      if (st == PI_OK && e == cudaSuccess && graph) {
        if (m->step_exec) {   // same topology as last time: new parameters into the old executable
          cudaGraphExecUpdateResultInfo info;
          if (cudaGraphExecUpdate(m->step_exec, graph, &info) != cudaSuccess) {
            cudaGetLastError();
            cudaGraphExecDestroy(m->step_exec);
            m->step_exec = nullptr;
          }
        }
        if (!m->step_exec) e = cudaGraphInstantiate(&m->step_exec, graph, 0);
      }
      if (st == PI_OK && e == cudaSuccess && m->step_exec) {
        for (; done < n_steps; ++done) {
          e = cudaGraphLaunch(m->step_exec, ctx->stream);
          if (e != cudaSuccess) break;
          ctx->launches += per_step;
        }
      }
      if (graph) cudaGraphDestroy(graph);
      if (st != PI_OK) return st;
    }
    if (e != cudaSuccess) {
      cudaGetLastError();  // fall back to eager launches for whatever is left
      ctx->err = std::string("CUDA graph path unavailable: ") + cudaGetErrorString(e);
    }
  }
  for (; done < n_steps; ++done) PI_TRY(decode_one_step(ctx, m, pool, batch, B, history, step_counter));
  PI_CUDA(ctx, cudaMemcpyAsync(out_tokens_host, history, (size_t)n_steps * B * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  return pi_ctx_synchronize(ctx);
}

pi_status pi_model_prefill(pi_ctx* ctx, pi_model* m, pi_kv_pool* pool, const uint32_t* tokens_host, int n, int start_pos,
                           const int32_t* block_table_host, int table_len, int chunk, float* last_logits_host_or_null,
                           uint32_t* argmax_host_or_null) {
  PI_ENTER(ctx);
  PI_REQUIRE(ctx, m && tokens_host, "null pointer");
  PI_REQUIRE(ctx, n > 0, "prefill needs at least one token");
  PI_REQUIRE(ctx, start_pos >= 0 && table_len >= 0, "negative start position or table length");
  PI_REQUIRE(ctx, block_table_host || table_len == 0, "null block table");
  PI_TRY(check_pool(ctx, m, pool));
  chunk = std::min(std::max(chunk, 1), m->capacity);  // clamp(1, capacity)
  std::vector<int32_t> tables, lens, pos;
  int last_rows = 0;
  for (int c0 = 0; c0 < n; c0 += chunk) {
    const int len = std::min(chunk, n - c0);
    tables.resize((size_t)len * std::max(table_len, 1));
    lens.assign(len, table_len);
    pos.resize(len);
    for (int i = 0; i < len; ++i) {
      pos[i] = start_pos + c0 + i;
      if (table_len) memcpy(&tables[(size_t)i * table_len], block_table_host, table_len * sizeof(int32_t));
    }
    pi_attn_batch batch;
    PI_TRY(stage_batch(ctx, m, pool, tokens_host + c0, pos.data(), tables.data(), table_len, lens.data(), len, &batch));
    PI_TRY(run_layers(ctx, m, pool, batch, len, nullptr));
    last_rows = len;
  }
  PI_TRY(project_logits(ctx, m, last_rows - 1, 1));
  PI_TRY(fetch_results(ctx, m, 1, last_logits_host_or_null, argmax_host_or_null));
  return pi_ctx_synchronize(ctx);
}

}  // extern "C"
