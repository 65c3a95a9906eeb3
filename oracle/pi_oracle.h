/*
 * CPU oracle for the int8 decode hot path of Paged-Infer.
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, in C++17, the reference's
 * CPU algorithms (Rust: src/math.rs, src/simd.rs, src/attention.rs,
 * src/memory/layout.rs, src/memory/block_table.rs, src/model.rs,
 * src/sampling.rs) so that the CUDA library can be checked against them.  It is
 * the checker and the timed CPU baseline; nothing in the product path links,
 * loads or calls it.
 *
 * Parity status: the reference is a Rust crate and cannot be compiled where
 * this oracle is built, so the restatement is pinned by (i) the reference's
 * golden fixture (NumPy HF-Llama logits, 40 x 112, tolerance 5e-4 and zero
 * argmax mismatches, tests/golden_parity_tests.rs:125-211), (ii) the
 * known-answer vectors of tests/math_tests.rs and (iii) the bit-identity
 * contracts of tests/simd_tests.rs and tests/attention_tests.rs.  int8 logits
 * have no golden file upstream: for those the parity is "pinned only by the
 * restatement".
 */
#ifndef PI_ORACLE_H
#define PI_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- simd.rs ------------------------------------------------------------ */
/* 1 when the AVX2+FMA kernels run, 0 for the portable scalar ones
 * (src/simd.rs:584-600). */
int orc_backend_avx2(void);
/* Force the scalar kernels (non-zero) or return to runtime dispatch (0). */
void orc_force_scalar(int on);
int orc_num_threads(void);
void orc_set_num_threads(int n);

float orc_dot_naive(const float* a, const float* b, size_t n);          /* src/simd.rs:26-33 */
float orc_dot_scalar(const float* a, const float* b, size_t n);         /* src/simd.rs:37-56 */
float orc_dot_i8_scalar(const int8_t* w, const float* x, size_t n);     /* src/simd.rs:60-77 */
float orc_dot(const float* a, const float* b, size_t n);                /* src/simd.rs:619-632 */
float orc_dot_i8(const int8_t* w, const float* x, size_t n);            /* src/simd.rs:635-648 */
/* out[j] = dot(w, x_block + j*stride) for j < bt, 1 <= bt <= 8
 * (src/simd.rs:694-726). */
void orc_dot_multi(const float* w, const float* x_block, size_t n, size_t stride, int bt, float* out);
void orc_dot_i8_multi(const int8_t* w, const float* x_block, size_t n, size_t stride, int bt, float* out);
void orc_axpy(float* out, float weight, const float* v, size_t n);      /* src/simd.rs:651-666 */

/* ---- math.rs ------------------------------------------------------------ */
void orc_quantize_rows_i8(const float* w, size_t rows, size_t cols, int8_t* q, float* scales); /* src/math.rs:456-469 */
void orc_matvec_i8(float* out, const float* x, const int8_t* w, const float* scales, size_t rows, size_t cols); /* :473-512 */
void orc_matvec_f32(float* out, const float* x, const float* w, size_t rows, size_t cols);     /* :93-129 */
void orc_matvec_f32_sequential(float* out, const float* x, const float* w, size_t rows, size_t cols); /* :73-86 */
/* out_rb is [row][batch]; tile is PAGED_INFER_MATMUL_TILE (4 by default). */
void orc_matmat_i8(float* out_rb, const float* x_br, const int8_t* w, const float* scales,
                   size_t batch, size_t rows, size_t cols, int tile);                           /* :223-275 */
void orc_matmat_f32(float* out_rb, const float* x_br, const float* w,
                    size_t batch, size_t rows, size_t cols, int tile);                          /* :164-220 */
void orc_transpose_rb_to_br(const float* src_rb, float* dst_br, size_t rows, size_t batch);    /* :281-290 */
void orc_pack_bf16_to_f32(const uint16_t* bf16, float* out, size_t n);                          /* :66-71 */
void orc_rms_norm(float* x, const float* weight, size_t n, float eps);                          /* :4-22 */
float orc_silu(float x);                                                                        /* :293-295 */
void orc_swiglu(float* x, const float* x_w3, size_t n);                                         /* :297-302 */
void orc_rope_table(size_t pos, size_t head_dim, float theta, float* cos_out, float* sin_out);  /* :331-341 */
/* style 0 = NeoX pairs (j, j+hd/2); 1 = interleaved pairs (2j, 2j+1). */
void orc_rope_rotate(float* x, size_t head_dim, const float* cos_t, const float* sin_t, int style); /* :344-367 */
void orc_softmax_in_place(float* x, size_t n);                                                  /* :405-426 */
size_t orc_argmax(const float* logits, size_t n);                                               /* src/sampling.rs:140-147 */

/* ---- memory/layout.rs --------------------------------------------------- */
typedef struct {
  int64_t num_layers, num_blocks, block_size, num_kv_heads, head_dim;
} orc_kv_layout;
size_t orc_kv_total_floats(const orc_kv_layout* l);
size_t orc_kv_index(const orc_kv_layout* l, size_t layer, size_t block, size_t tok, size_t kv_head, int is_value);
/* returns 0, or -1 when src == dst (the reference asserts). */
int orc_kv_copy_block(const orc_kv_layout* l, float* cache, size_t src, size_t dst);

/* ---- attention.rs ------------------------------------------------------- */
/* Block tables are rows of a [B x max_blocks] int32 matrix; table_lens[b] is
 * the number of mapped logical blocks (BlockTable::len()). */
size_t orc_lane_width(size_t kv_group, size_t num_kv_heads, size_t batch, size_t threads, size_t lanes_per_thread);
/* returns 0 or -1 on a violated shape assertion (src/attention.rs:159-180). */
int orc_paged_attention_run(float* out, float* scores, const float* q, const float* kv_cache,
                            const orc_kv_layout* layout, size_t block_size, size_t num_heads,
                            size_t head_dim, size_t kv_group, size_t score_stride, size_t heads_per_lane,
                            const int32_t* tables, size_t max_blocks, const int32_t* table_lens,
                            const int64_t* pos, const int64_t* start, size_t batch, size_t layer);

/* ---- model.rs ----------------------------------------------------------- */
enum { ORC_F32 = 0, ORC_INT8 = 1, ORC_BF16 = 2 };
typedef struct {
  int32_t kind;          /* ORC_F32 / ORC_INT8 / ORC_BF16 (widened to f32 at load) */
  int64_t rows, cols;
  const void* data;      /* f32 / int8 / bf16 bits, row-major [rows][cols] */
  const float* scales;   /* int8 only: [rows] */
} orc_tensor;

typedef struct {
  int64_t hidden_size, num_hidden_layers, num_attention_heads, num_key_value_heads;
  int64_t intermediate_size, vocab_size;
  float rms_norm_eps, rope_theta;
  int64_t attention_window;   /* < 0: none */
  int32_t rope_style;         /* 0 NeoX, 1 interleaved */
} orc_model_config;

typedef struct {
  const uint16_t* token_embeddings_bf16;  /* [vocab][hidden] */
  const float* final_norm;                /* [hidden] */
  const float* const* attention_norm;     /* [layers] -> [hidden] */
  const float* const* ffn_norm;           /* [layers] -> [hidden] */
  /* [layers*7]: wq, wk, wv, wo, w1 (gate), w2 (down), w3 (up) */
  const orc_tensor* projections;
  orc_tensor lm_head;
} orc_model_weights;

typedef struct orc_model orc_model;
orc_model* orc_model_create(const orc_model_config* cfg, const orc_model_weights* w);
void orc_model_destroy(orc_model* m);
size_t orc_model_weight_bytes(const orc_model* m);

/* LlamaWeights::forward_into (src/model.rs:659-681): one token, logits[vocab]. */
int orc_model_forward(orc_model* m, uint32_t token, size_t pos, const int32_t* table, size_t table_len,
                      float* kv_cache, size_t kv_len, size_t block_size, float* logits);
/* LlamaWeights::prefill_into (:726-751): token by token, last logits. */
int orc_model_prefill(orc_model* m, const uint32_t* tokens, size_t n, size_t start_pos,
                      const int32_t* table, size_t table_len, float* kv_cache, size_t kv_len,
                      size_t block_size, float* logits);
/* LlamaWeights::decode_batch_into (:1184-1207): logits [batch][vocab]. */
int orc_model_decode_batch(orc_model* m, const uint32_t* tokens, const int64_t* positions,
                           const int32_t* tables, size_t max_blocks, const int32_t* table_lens,
                           size_t batch, float* kv_cache, size_t kv_len, size_t block_size, float* logits);
/* LlamaWeights::prefill_batched (:1222-1255): logits[vocab] of the last position. */
int orc_model_prefill_batched(orc_model* m, const uint32_t* tokens, size_t n, size_t start_pos,
                              const int32_t* table, size_t table_len, float* kv_cache, size_t kv_len,
                              size_t block_size, size_t chunk_size, size_t capacity, float* logits);

#ifdef __cplusplus
}
#endif
#endif
