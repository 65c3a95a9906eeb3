// CPU oracle: a C++17 restatement of the reference's CPU kernels and forward
// pass.  TEST INFRASTRUCTURE ONLY - see pi_oracle.h for what pins it and who may
// call it.  Each function names the reference file:line it follows.
//
// Float semantics that matter for bit-level agreement with the reference on an
// x86-64 host:
//   * The AVX2+FMA kernels keep four 8-lane accumulators, chunk 32 elements,
//     then 8-element chunks into accumulator 0, reduce (a0+a1)+(a2+a3), do the
//     horizontal sum as (lo+hi) -> (+movehl) -> (+lane 1), and add the scalar
//     remainder last in index order (src/simd.rs:100-262).
//   * Scalar code must not be contracted into FMAs or re-associated, so this
//     file is compiled with -ffp-contract=off and without -ffast-math.
//   * exp/pow/sin/cos/sqrt are the platform libm's f32 routines, which is what
//     Rust's f32 methods lower to on Linux.
#include "pi_oracle.h"

#include <immintrin.h>
#include <math.h>
#include <string.h>

#include <algorithm>
#include <memory>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

bool g_force_scalar = false;

bool cpu_has_avx2_fma() {
  static const bool ok = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  return ok;
}
inline bool use_avx2() { return !g_force_scalar && cpu_has_avx2_fma(); }

// ---- scalar kernels (src/simd.rs:26-85) -----------------------------------

template <class W>
float dot4_scalar(const W* w, const float* x, size_t n) {
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  size_t i = 0;
  for (; i + 4 <= n; i += 4) {
    acc[0] += (float)w[i] * x[i];
    acc[1] += (float)w[i + 1] * x[i + 1];
    acc[2] += (float)w[i + 2] * x[i + 2];
    acc[3] += (float)w[i + 3] * x[i + 3];
  }
  float total = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  for (; i < n; ++i) total += (float)w[i] * x[i];
  return total;
}

// ---- AVX2 + FMA kernels (src/simd.rs:89-350) ------------------------------

#define ORC_AVX2 __attribute__((target("avx2,fma")))

ORC_AVX2 inline __m256 widen8(const float* p) { return _mm256_loadu_ps(p); }
ORC_AVX2 inline __m256 widen8(const int8_t* p) {
  // 8 bytes -> sign-extended i32 lanes -> f32 (src/simd.rs:237-240)
  return _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)p)));
}

ORC_AVX2 inline float hsum8(__m256 v) {  // src/simd.rs:100-109
  __m128 lo = _mm256_castps256_ps128(v);
  __m128 hi = _mm256_extractf128_ps(v, 1);
  __m128 s = _mm_add_ps(lo, hi);
  s = _mm_add_ps(s, _mm_movehl_ps(s, s));
  s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 0x55));
  return _mm_cvtss_f32(s);
}

// One weight row against BT activation rows.  BT == 1 is the plain dot; the
// accumulator structure is shared so every BT gives the same bits per output
// (src/simd.rs:172-217 for f32 weights, :279-329 for int8 weights).
template <class W, int BT>
ORC_AVX2 void dot_multi_avx2(const W* w, const float* xb, size_t n, size_t stride, float* out) {
  __m256 acc[BT][4];
  for (int b = 0; b < BT; ++b)
    for (int j = 0; j < 4; ++j) acc[b][j] = _mm256_setzero_ps();

  size_t i = 0;
  for (; i + 32 <= n; i += 32) {
    for (int j = 0; j < 4; ++j) {
      const __m256 wv = widen8(w + i + 8 * j);
      for (int b = 0; b < BT; ++b)
        acc[b][j] = _mm256_fmadd_ps(wv, _mm256_loadu_ps(xb + b * stride + i + 8 * j), acc[b][j]);
    }
  }
  for (; i + 8 <= n; i += 8) {
    const __m256 wv = widen8(w + i);
    for (int b = 0; b < BT; ++b)
      acc[b][0] = _mm256_fmadd_ps(wv, _mm256_loadu_ps(xb + b * stride + i), acc[b][0]);
  }
  for (int b = 0; b < BT; ++b) {
    __m256 sum = _mm256_add_ps(_mm256_add_ps(acc[b][0], acc[b][1]), _mm256_add_ps(acc[b][2], acc[b][3]));
    float total = hsum8(sum);
    for (size_t k = i; k < n; ++k) total += (float)w[k] * xb[b * stride + k];
    out[b] = total;
  }
}

template <class W>
void dot_multi_any(const W* w, const float* xb, size_t n, size_t stride, int bt, float* out) {
  if (use_avx2()) {
    switch (bt) {
      case 1: dot_multi_avx2<W, 1>(w, xb, n, stride, out); return;
      case 2: dot_multi_avx2<W, 2>(w, xb, n, stride, out); return;
      case 3: dot_multi_avx2<W, 3>(w, xb, n, stride, out); return;
      case 4: dot_multi_avx2<W, 4>(w, xb, n, stride, out); return;
      case 5: dot_multi_avx2<W, 5>(w, xb, n, stride, out); return;
      case 6: dot_multi_avx2<W, 6>(w, xb, n, stride, out); return;
      case 7: dot_multi_avx2<W, 7>(w, xb, n, stride, out); return;
      case 8: dot_multi_avx2<W, 8>(w, xb, n, stride, out); return;
      default: break;
    }
  }
  // Portable: literally bt scalar dots (src/simd.rs:709-711, :725).
  for (int b = 0; b < bt; ++b) out[b] = dot4_scalar(w, xb + (size_t)b * stride, n);
}

template <class W>
inline float dot_any(const W* w, const float* x, size_t n) {
  float r;
  dot_multi_any(w, x, n, n, 1, &r);
  return r;
}

ORC_AVX2 void axpy_avx2(float* out, float weight, const float* v, size_t n) {  // src/simd.rs:334-349
  const __m256 w = _mm256_set1_ps(weight);
  size_t i = 0;
  for (; i + 8 <= n; i += 8)
    _mm256_storeu_ps(out + i, _mm256_fmadd_ps(w, _mm256_loadu_ps(v + i), _mm256_loadu_ps(out + i)));
  for (; i < n; ++i) out[i] += weight * v[i];
}

inline void axpy_any(float* out, float weight, const float* v, size_t n) {
  if (use_avx2()) {
    axpy_avx2(out, weight, v, n);
    return;
  }
  for (size_t i = 0; i < n; ++i) out[i] += weight * v[i];  // src/simd.rs:81-85
}

// ---- batched row kernel (src/math.rs:164-275) ------------------------------
// One weight row against every batch entry: tiles of 4, then 2, then 1.
template <class W>
inline void row_times_batch(const W* w_row, const float* x_br, size_t batch, size_t cols, int tile,
                            float scale, bool scaled, float* out_row) {
  size_t b = 0;
  float got[4];
  if (tile >= 4) {
    for (; b + 4 <= batch; b += 4) {
      dot_multi_any(w_row, x_br + b * cols, cols, cols, 4, got);
      for (int j = 0; j < 4; ++j) out_row[b + j] = scaled ? got[j] * scale : got[j];
    }
  }
  if (tile >= 2) {
    for (; b + 2 <= batch; b += 2) {
      dot_multi_any(w_row, x_br + b * cols, cols, cols, 2, got);
      for (int j = 0; j < 2; ++j) out_row[b + j] = scaled ? got[j] * scale : got[j];
    }
  }
  for (; b < batch; ++b) {
    float d = dot_any(w_row, x_br + b * cols, cols);
    out_row[b] = scaled ? d * scale : d;
  }
}

inline float bf16_to_f32(uint16_t bits) {  // half::bf16::to_f32 - an exact 16-bit shift
  uint32_t u = (uint32_t)bits << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

}  // namespace

// ===========================================================================
// simd.rs
// ===========================================================================
extern "C" {

int orc_backend_avx2(void) { return use_avx2() ? 1 : 0; }
void orc_force_scalar(int on) { g_force_scalar = on != 0; }
int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

float orc_dot_naive(const float* a, const float* b, size_t n) {
  float acc = 0.f;
  for (size_t i = 0; i < n; ++i) acc += a[i] * b[i];
  return acc;
}
float orc_dot_scalar(const float* a, const float* b, size_t n) { return dot4_scalar(a, b, n); }
float orc_dot_i8_scalar(const int8_t* w, const float* x, size_t n) { return dot4_scalar(w, x, n); }
float orc_dot(const float* a, const float* b, size_t n) { return dot_any(a, b, n); }
float orc_dot_i8(const int8_t* w, const float* x, size_t n) { return dot_any(w, x, n); }
void orc_dot_multi(const float* w, const float* xb, size_t n, size_t stride, int bt, float* out) {
  dot_multi_any(w, xb, std::min(n, stride), stride, bt, out);
}
void orc_dot_i8_multi(const int8_t* w, const float* xb, size_t n, size_t stride, int bt, float* out) {
  dot_multi_any(w, xb, std::min(n, stride), stride, bt, out);
}
void orc_axpy(float* out, float weight, const float* v, size_t n) { axpy_any(out, weight, v, n); }

// ===========================================================================
// math.rs
// ===========================================================================

// src/math.rs:456-469.  scale = absmax/127 (1.0 for an all-zero row); code =
// round-half-away(w / scale) clamped to +-127, with a true IEEE division.
void orc_quantize_rows_i8(const float* w, size_t rows, size_t cols, int8_t* q, float* scales) {
  for (size_t r = 0; r < rows; ++r) {
    const float* row = w + r * cols;
    float max_abs = 0.f;
    // f32::max ignores a NaN operand; fmaxf has the same rule.
    for (size_t c = 0; c < cols; ++c) max_abs = fmaxf(max_abs, fabsf(row[c]));
    const float scale = max_abs > 0.f ? max_abs / 127.0f : 1.0f;
    scales[r] = scale;
    for (size_t c = 0; c < cols; ++c) {
      float v = roundf(row[c] / scale);
      // f32::clamp keeps NaN; `as i8` then maps NaN to 0 and saturates.
      if (v < -127.f) v = -127.f;
      if (v > 127.f) v = 127.f;
      q[r * cols + c] = (v != v) ? (int8_t)0 : (int8_t)v;
    }
  }
}

void orc_matvec_i8(float* out, const float* x, const int8_t* w, const float* scales, size_t rows, size_t cols) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; ++r) out[r] = dot_any(w + (size_t)r * cols, x, cols) * scales[r];
}

void orc_matvec_f32(float* out, const float* x, const float* w, size_t rows, size_t cols) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; ++r) out[r] = dot_any(w + (size_t)r * cols, x, cols);
}

void orc_matvec_f32_sequential(float* out, const float* x, const float* w, size_t rows, size_t cols) {
  for (size_t r = 0; r < rows; ++r) out[r] = orc_dot_naive(w + r * cols, x, cols);
}

void orc_matmat_i8(float* out_rb, const float* x_br, const int8_t* w, const float* scales,
                   size_t batch, size_t rows, size_t cols, int tile) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; ++r)
    row_times_batch(w + (size_t)r * cols, x_br, batch, cols, tile, scales[r], true, out_rb + (size_t)r * batch);
}

void orc_matmat_f32(float* out_rb, const float* x_br, const float* w, size_t batch, size_t rows, size_t cols, int tile) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; ++r)
    row_times_batch(w + (size_t)r * cols, x_br, batch, cols, tile, 1.0f, false, out_rb + (size_t)r * batch);
}

void orc_transpose_rb_to_br(const float* src_rb, float* dst_br, size_t rows, size_t batch) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t b = 0; b < batch; ++b) dst_br[b * rows + r] = src_rb[r * batch + b];
}

void orc_pack_bf16_to_f32(const uint16_t* bf16, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = bf16_to_f32(bf16[i]);
}

void orc_rms_norm(float* x, const float* weight, size_t n, float eps) {
  float ss = 0.f;
  for (size_t i = 0; i < n; ++i) ss += x[i] * x[i];
  ss /= (float)n;
  const float inv_norm = 1.0f / sqrtf(ss + eps);
  for (size_t i = 0; i < n; ++i) x[i] = x[i] * inv_norm * weight[i];
}

float orc_silu(float x) { return x / (1.0f + expf(-x)); }

void orc_swiglu(float* x, const float* x_w3, size_t n) {
  for (size_t i = 0; i < n; ++i) x[i] = orc_silu(x[i]) * x_w3[i];
}

void orc_rope_table(size_t pos, size_t head_dim, float theta, float* cos_out, float* sin_out) {
  const size_t half = head_dim / 2;
  for (size_t j = 0; j < half; ++j) {
    const float freq = 1.0f / powf(theta, (float)(2 * j) / (float)head_dim);
    const float a = (float)pos * freq;
    sin_out[j] = sinf(a);
    cos_out[j] = cosf(a);
  }
}

void orc_rope_rotate(float* x, size_t head_dim, const float* c, const float* s, int style) {
  const size_t half = head_dim / 2;
  if (style == 0) {
    for (size_t j = 0; j < half; ++j) {
      const float a = x[j], b = x[j + half];
      x[j] = a * c[j] - b * s[j];
      x[j + half] = b * c[j] + a * s[j];
    }
  } else {
    for (size_t j = 0; j < half; ++j) {
      const float a = x[2 * j], b = x[2 * j + 1];
      x[2 * j] = a * c[j] - b * s[j];
      x[2 * j + 1] = b * c[j] + a * s[j];
    }
  }
}

void orc_softmax_in_place(float* x, size_t n) {
  if (n == 0) return;
  float max_v = -INFINITY;
  for (size_t i = 0; i < n; ++i) max_v = fmaxf(max_v, x[i]);
  if (!isfinite(max_v)) {  // every entry masked: zeros, not NaN
    for (size_t i = 0; i < n; ++i) x[i] = 0.f;
    return;
  }
  float sum = 0.f;
  for (size_t i = 0; i < n; ++i) {
    x[i] = expf(x[i] - max_v);
    sum += x[i];
  }
  const float inv_sum = 1.0f / fmaxf(sum, 1e-12f);
  for (size_t i = 0; i < n; ++i) x[i] *= inv_sum;
}

// Iterator::max_by(total_cmp) keeps the LAST maximal element.
size_t orc_argmax(const float* logits, size_t n) {
  if (n == 0) return 0;
  auto key = [](float f) {  // f32::total_cmp ordering as a signed integer key
    int32_t b;
    memcpy(&b, &f, 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
  };
  size_t best = 0;
  int32_t best_key = key(logits[0]);
  for (size_t i = 1; i < n; ++i) {
    const int32_t k = key(logits[i]);
    if (k >= best_key) {
      best_key = k;
      best = i;
    }
  }
  return best;
}

// ===========================================================================
// memory/layout.rs
// ===========================================================================
size_t orc_kv_total_floats(const orc_kv_layout* l) {
  return (size_t)l->num_layers * l->num_blocks * l->block_size * l->num_kv_heads * 2 * l->head_dim;
}
static inline size_t kv_block_stride(const orc_kv_layout* l) {
  return (size_t)l->block_size * l->num_kv_heads * 2 * l->head_dim;
}
size_t orc_kv_index(const orc_kv_layout* l, size_t layer, size_t block, size_t tok, size_t kv_head, int is_value) {
  return ((((layer * l->num_blocks + block) * l->block_size + tok) * l->num_kv_heads + kv_head) * 2 +
          (is_value ? 1 : 0)) * l->head_dim;
}
int orc_kv_copy_block(const orc_kv_layout* l, float* cache, size_t src, size_t dst) {
  if (src == dst) return -1;
  const size_t bs = kv_block_stride(l);
  for (size_t layer = 0; layer < (size_t)l->num_layers; ++layer) {
    const float* s = cache + (layer * l->num_blocks + src) * bs;
    float* d = cache + (layer * l->num_blocks + dst) * bs;
    memcpy(d, s, bs * sizeof(float));
  }
  return 0;
}

// ===========================================================================
// attention.rs
// ===========================================================================
size_t orc_lane_width(size_t kv_group, size_t num_kv_heads, size_t batch, size_t threads, size_t lanes_per_thread) {
  const size_t want = std::max<size_t>(threads, 1) * lanes_per_thread;  // src/attention.rs:126-132
  for (size_t d = std::max<size_t>(kv_group, 1); d >= 1; --d)
    if (kv_group % d == 0 && batch * num_kv_heads * (kv_group / d) >= want) return d;
  return 1;
}
}  // extern "C"

namespace {
struct Entry {
  const int32_t* table;
  size_t table_len;
  size_t pos, start;
  size_t window_len() const { return pos + 1 > start ? pos + 1 - start : 0; }
};

// Walk the attended window one logical block at a time
// (src/attention.rs:279-295): f(score_offset, first_offset, take, block|-1).
template <class F>
inline void for_each_block(const Entry& e, size_t block_size, F&& f) {
  size_t t = e.start;
  while (t <= e.pos) {
    const size_t first_offset = t % block_size;
    const size_t take = std::min(block_size - first_offset, e.pos + 1 - t);
    const size_t lb = t / block_size;
    const long block = lb < e.table_len ? (long)e.table[lb] : -1;  // BlockTable::get_physical_location
    f(t - e.start, first_offset, take, block);
    t += take;
  }
}

int attention_run(float* out, float* scores, const float* q, const float* kv, const orc_kv_layout& L,
                  size_t block_size, size_t num_heads, size_t head_dim, size_t kv_group, size_t score_stride,
                  size_t d, const std::vector<Entry>& entries, size_t layer) {
  const size_t batch = entries.size();
  if (!(kv_group > 0 && num_heads == kv_group * (size_t)L.num_kv_heads)) return -1;
  if (!(d > 0 && kv_group % d == 0)) return -1;
  if (!(batch == 0 || score_stride > 0)) return -1;
  const float scale = 1.0f / sqrtf((float)head_dim);
  const size_t lanes_per_entry = num_heads / d;
  const size_t token_stride = (size_t)L.num_kv_heads * 2 * head_dim;
  const long lanes = (long)(batch * lanes_per_entry);

#pragma omp parallel for schedule(dynamic, 1)
  for (long lane = 0; lane < lanes; ++lane) {
    const Entry& e = entries[lane / lanes_per_entry];
    const size_t h0 = (lane % lanes_per_entry) * d;
    const size_t kv_h = h0 / kv_group;
    const float* q_lane = q + (size_t)lane * d * head_dim;
    float* out_lane = out + (size_t)lane * d * head_dim;
    float* score_lane = scores + (size_t)lane * d * score_stride;
    const size_t used = e.window_len();
    if (used == 0) {
      std::fill(out_lane, out_lane + d * head_dim, 0.f);
      continue;
    }
    for_each_block(e, block_size, [&](size_t si0, size_t first, size_t take, long block) {
      if (block >= 0) {
        const size_t base = orc_kv_index(&L, layer, (size_t)block, first, kv_h, 0);
        for (size_t i = 0; i < take; ++i) {
          const float* k = kv + base + i * token_stride;
          for (size_t g = 0; g < d; ++g)
            score_lane[g * score_stride + si0 + i] = dot_any(q_lane + g * head_dim, k, head_dim) * scale;
        }
      } else {
        for (size_t g = 0; g < d; ++g)
          std::fill(score_lane + g * score_stride + si0, score_lane + g * score_stride + si0 + take, -INFINITY);
      }
    });
    for (size_t g = 0; g < d; ++g) orc_softmax_in_place(score_lane + g * score_stride, used);
    std::fill(out_lane, out_lane + d * head_dim, 0.f);
    for_each_block(e, block_size, [&](size_t si0, size_t first, size_t take, long block) {
      if (block < 0) return;
      const size_t base = orc_kv_index(&L, layer, (size_t)block, first, kv_h, 1);
      for (size_t i = 0; i < take; ++i) {
        const float* v = kv + base + i * token_stride;
        for (size_t g = 0; g < d; ++g) {
          const float w = score_lane[g * score_stride + si0 + i];
          if (w == 0.0f) continue;
          axpy_any(out_lane + g * head_dim, w, v, head_dim);
        }
      }
    });
  }
  return 0;
}
}  // namespace

extern "C" {
int orc_paged_attention_run(float* out, float* scores, const float* q, const float* kv_cache,
                            const orc_kv_layout* layout, size_t block_size, size_t num_heads, size_t head_dim,
                            size_t kv_group, size_t score_stride, size_t heads_per_lane, const int32_t* tables,
                            size_t max_blocks, const int32_t* table_lens, const int64_t* pos,
                            const int64_t* start, size_t batch, size_t layer) {
  std::vector<Entry> entries(batch);
  for (size_t b = 0; b < batch; ++b)
    entries[b] = Entry{tables + b * max_blocks, (size_t)table_lens[b], (size_t)pos[b], (size_t)start[b]};
  return attention_run(out, scores, q, kv_cache, *layout, block_size, num_heads, head_dim, kv_group,
                       score_stride, heads_per_lane, entries, layer);
}

// ===========================================================================
// model.rs
// ===========================================================================
}  // extern "C"

namespace {
struct Linear {  // Projection::{F32, Int8} (src/model.rs:218-291)
  bool int8 = false;
  size_t rows = 0, cols = 0;
  std::vector<float> w;
  std::vector<int8_t> q;
  std::vector<float> scales;

  void load(const orc_tensor& t) {
    rows = (size_t)t.rows;
    cols = (size_t)t.cols;
    const size_t n = rows * cols;
    if (t.kind == ORC_INT8) {
      int8 = true;
      q.assign((const int8_t*)t.data, (const int8_t*)t.data + n);
      scales.assign(t.scales, t.scales + rows);
    } else if (t.kind == ORC_BF16) {
      w.resize(n);
      orc_pack_bf16_to_f32((const uint16_t*)t.data, w.data(), n);
    } else {
      w.assign((const float*)t.data, (const float*)t.data + n);
    }
  }
  void apply_parallel(float* out, const float* x) const {
    if (int8) orc_matvec_i8(out, x, q.data(), scales.data(), rows, cols);
    else orc_matvec_f32(out, x, w.data(), rows, cols);
  }
  // apply_batched (src/model.rs:247-259): [row][batch] into stage, then transpose.
  void apply_batched(float* out_br, const float* x_br, size_t batch, float* stage) const {
    if (int8) orc_matmat_i8(stage, x_br, q.data(), scales.data(), batch, rows, cols, 4);
    else orc_matmat_f32(stage, x_br, w.data(), batch, rows, cols, 4);
    orc_transpose_rb_to_br(stage, out_br, rows, batch);
  }
  size_t weight_bytes() const { return int8 ? q.size() + 4 * scales.size() : 4 * w.size(); }
};

struct Layer {
  std::vector<float> attention_norm, ffn_norm;
  Linear wq, wk, wv, wo, w1, w2, w3;
};
}  // namespace

struct orc_model {
  orc_model_config cfg;
  std::vector<uint16_t> embed;
  std::vector<float> final_norm;
  std::vector<Layer> layers;
  Linear lm_head;

  size_t head_dim() const { return (size_t)(cfg.hidden_size / cfg.num_attention_heads); }
  size_t kv_group() const { return (size_t)(cfg.num_attention_heads / cfg.num_key_value_heads); }
  size_t kv_dim() const { return (size_t)cfg.num_key_value_heads * head_dim(); }
  orc_kv_layout layout_for_cache(size_t cache_len, size_t block_size) const {  // src/model.rs:133-137
    const size_t per_block = (size_t)cfg.num_hidden_layers * block_size * cfg.num_key_value_heads * 2 * head_dim();
    orc_kv_layout l;
    l.num_layers = cfg.num_hidden_layers;
    l.num_blocks = (int64_t)(cache_len / std::max<size_t>(per_block, 1));
    l.block_size = (int64_t)block_size;
    l.num_kv_heads = cfg.num_key_value_heads;
    l.head_dim = (int64_t)head_dim();
    return l;
  }
};

namespace {

inline size_t window_start(size_t pos, int64_t window) {  // AttnEntry::new (src/attention.rs:71-78)
  if (window < 0) return 0;
  const size_t w = (size_t)window;
  return pos + 1 > w ? pos + 1 - w : 0;
}

// run_layers_batch (src/model.rs:968-1177).  Leaves the final normalised hidden
// state of every entry in x[batch][hidden].
void run_layers_batch(const orc_model& m, const uint32_t* tokens, const size_t* positions,
                      const std::vector<Entry>& tables_in, size_t batch, float* kv, size_t kv_len,
                      size_t block_size, std::vector<float>& x) {
  const orc_model_config& c = m.cfg;
  const size_t hidden = (size_t)c.hidden_size, head_dim = m.head_dim(), kv_dim = m.kv_dim();
  const size_t inter = (size_t)c.intermediate_size, num_heads = (size_t)c.num_attention_heads;
  const size_t num_kv_heads = (size_t)c.num_key_value_heads, kv_group = m.kv_group(), half = head_dim / 2;
  const orc_kv_layout L = m.layout_for_cache(kv_len, block_size);

  std::vector<float> rope_cos(batch * half), rope_sin(batch * half);
  std::vector<Entry> entries(batch);
  size_t widest = 0;
  for (size_t b = 0; b < batch; ++b) {
    orc_rope_table(positions[b], head_dim, c.rope_theta, &rope_cos[b * half], &rope_sin[b * half]);
    entries[b] = tables_in[b];
    entries[b].pos = positions[b];
    entries[b].start = window_start(positions[b], c.attention_window);
    widest = std::max(widest, entries[b].window_len());
  }
  widest = std::max<size_t>(widest, 1);

  x.assign(batch * hidden, 0.f);
  for (size_t b = 0; b < batch; ++b) {
    const size_t token = (size_t)tokens[b] % (size_t)c.vocab_size;
    orc_pack_bf16_to_f32(&m.embed[token * hidden], &x[b * hidden], hidden);
  }

  const size_t widest_rows = std::max({(size_t)c.vocab_size, inter, hidden, kv_dim});
  std::vector<float> xb(batch * hidden), attn_out(batch * hidden), proj_out(batch * hidden), q(batch * hidden);
  std::vector<float> k(batch * kv_dim), v(batch * kv_dim), ff_gate(batch * inter), ff_up(batch * inter);
  std::vector<float> ff_down(batch * hidden), stage(batch * widest_rows), scores(batch * num_heads * widest);
  const size_t d = orc_lane_width(kv_group, num_kv_heads, batch, (size_t)orc_num_threads(), 2);

  for (size_t li = 0; li < m.layers.size(); ++li) {
    const Layer& layer = m.layers[li];
    for (size_t b = 0; b < batch; ++b) {
      std::copy(&x[b * hidden], &x[(b + 1) * hidden], &xb[b * hidden]);
      orc_rms_norm(&xb[b * hidden], layer.attention_norm.data(), hidden, c.rms_norm_eps);
    }
    layer.wq.apply_batched(q.data(), xb.data(), batch, stage.data());
    layer.wk.apply_batched(k.data(), xb.data(), batch, stage.data());
    layer.wv.apply_batched(v.data(), xb.data(), batch, stage.data());

    for (size_t b = 0; b < batch; ++b) {
      const float* cs = &rope_cos[b * half];
      const float* sn = &rope_sin[b * half];
      for (size_t h = 0; h < num_heads; ++h) orc_rope_rotate(&q[b * hidden + h * head_dim], head_dim, cs, sn, c.rope_style);
      for (size_t h = 0; h < num_kv_heads; ++h) orc_rope_rotate(&k[b * kv_dim + h * head_dim], head_dim, cs, sn, c.rope_style);
    }
    for (size_t b = 0; b < batch; ++b) {  // K/V scatter; silently skipped when unmapped
      const size_t lb = positions[b] / block_size, off = positions[b] % block_size;
      if (lb >= entries[b].table_len) continue;
      const size_t pb = (size_t)entries[b].table[lb];
      for (size_t h = 0; h < num_kv_heads; ++h) {
        const size_t src = b * kv_dim + h * head_dim;
        std::copy(&k[src], &k[src + head_dim], kv + orc_kv_index(&L, li, pb, off, h, 0));
        std::copy(&v[src], &v[src + head_dim], kv + orc_kv_index(&L, li, pb, off, h, 1));
      }
    }
    attention_run(attn_out.data(), scores.data(), q.data(), kv, L, block_size, num_heads, head_dim, kv_group,
                  widest, d, entries, li);

    layer.wo.apply_batched(proj_out.data(), attn_out.data(), batch, stage.data());
    for (size_t i = 0; i < batch * hidden; ++i) x[i] += proj_out[i];

    for (size_t b = 0; b < batch; ++b) {
      std::copy(&x[b * hidden], &x[(b + 1) * hidden], &xb[b * hidden]);
      orc_rms_norm(&xb[b * hidden], layer.ffn_norm.data(), hidden, c.rms_norm_eps);
    }
    layer.w1.apply_batched(ff_gate.data(), xb.data(), batch, stage.data());
    layer.w3.apply_batched(ff_up.data(), xb.data(), batch, stage.data());
    orc_swiglu(ff_gate.data(), ff_up.data(), batch * inter);
    layer.w2.apply_batched(ff_down.data(), ff_gate.data(), batch, stage.data());
    for (size_t i = 0; i < batch * hidden; ++i) x[i] += ff_down[i];
  }
  for (size_t b = 0; b < batch; ++b) orc_rms_norm(&x[b * hidden], m.final_norm.data(), hidden, c.rms_norm_eps);
}

// run_layers (src/model.rs:770-940): the single-token path, matvec kernels and a
// batch-of-one attention call.
void run_layers(const orc_model& m, uint32_t token_id, size_t pos, const Entry& table, float* kv, size_t kv_len,
                size_t block_size, std::vector<float>& x) {
  const orc_model_config& c = m.cfg;
  const size_t hidden = (size_t)c.hidden_size, head_dim = m.head_dim(), kv_dim = m.kv_dim();
  const size_t inter = (size_t)c.intermediate_size, num_heads = (size_t)c.num_attention_heads;
  const size_t num_kv_heads = (size_t)c.num_key_value_heads, kv_group = m.kv_group(), half = head_dim / 2;
  const orc_kv_layout L = m.layout_for_cache(kv_len, block_size);

  std::vector<Entry> entry(1, table);
  entry[0].pos = pos;
  entry[0].start = window_start(pos, c.attention_window);
  const size_t window_len = std::max<size_t>(entry[0].window_len(), 1);
  const size_t d = orc_lane_width(kv_group, num_kv_heads, 1, (size_t)orc_num_threads(), 2);

  std::vector<float> rope_cos(half), rope_sin(half);
  orc_rope_table(pos, head_dim, c.rope_theta, rope_cos.data(), rope_sin.data());

  x.assign(hidden, 0.f);
  const size_t token = (size_t)token_id % (size_t)c.vocab_size;
  orc_pack_bf16_to_f32(&m.embed[token * hidden], x.data(), hidden);

  std::vector<float> xb(hidden), attn_out(hidden), proj_out(hidden), q(hidden), k(kv_dim), v(kv_dim);
  std::vector<float> ff_gate(inter), ff_up(inter), ff_down(hidden), scores(num_heads * window_len);

  for (size_t li = 0; li < m.layers.size(); ++li) {
    const Layer& layer = m.layers[li];
    xb = x;
    orc_rms_norm(xb.data(), layer.attention_norm.data(), hidden, c.rms_norm_eps);
    layer.wq.apply_parallel(q.data(), xb.data());
    layer.wk.apply_parallel(k.data(), xb.data());
    layer.wv.apply_parallel(v.data(), xb.data());
    for (size_t h = 0; h < num_heads; ++h) orc_rope_rotate(&q[h * head_dim], head_dim, rope_cos.data(), rope_sin.data(), c.rope_style);
    for (size_t h = 0; h < num_kv_heads; ++h) orc_rope_rotate(&k[h * head_dim], head_dim, rope_cos.data(), rope_sin.data(), c.rope_style);
    const size_t lb = pos / block_size, off = pos % block_size;
    if (lb < table.table_len) {
      const size_t pb = (size_t)table.table[lb];
      for (size_t h = 0; h < num_kv_heads; ++h) {
        std::copy(&k[h * head_dim], &k[(h + 1) * head_dim], kv + orc_kv_index(&L, li, pb, off, h, 0));
        std::copy(&v[h * head_dim], &v[(h + 1) * head_dim], kv + orc_kv_index(&L, li, pb, off, h, 1));
      }
    }
    attention_run(attn_out.data(), scores.data(), q.data(), kv, L, block_size, num_heads, head_dim, kv_group,
                  window_len, d, entry, li);
    layer.wo.apply_parallel(proj_out.data(), attn_out.data());
    for (size_t i = 0; i < hidden; ++i) x[i] += proj_out[i];
    xb = x;
    orc_rms_norm(xb.data(), layer.ffn_norm.data(), hidden, c.rms_norm_eps);
    layer.w1.apply_parallel(ff_gate.data(), xb.data());
    layer.w3.apply_parallel(ff_up.data(), xb.data());
    orc_swiglu(ff_gate.data(), ff_up.data(), inter);
    layer.w2.apply_parallel(ff_down.data(), ff_gate.data());
    for (size_t i = 0; i < hidden; ++i) x[i] += ff_down[i];
  }
  orc_rms_norm(x.data(), m.final_norm.data(), hidden, c.rms_norm_eps);
}

}  // namespace

extern "C" {

orc_model* orc_model_create(const orc_model_config* cfg, const orc_model_weights* w) {
  auto m = std::make_unique<orc_model>();
  m->cfg = *cfg;
  const size_t hidden = (size_t)cfg->hidden_size, vocab = (size_t)cfg->vocab_size, nl = (size_t)cfg->num_hidden_layers;
  m->embed.assign(w->token_embeddings_bf16, w->token_embeddings_bf16 + vocab * hidden);
  m->final_norm.assign(w->final_norm, w->final_norm + hidden);
  m->layers.resize(nl);
  for (size_t l = 0; l < nl; ++l) {
    Layer& L = m->layers[l];
    L.attention_norm.assign(w->attention_norm[l], w->attention_norm[l] + hidden);
    L.ffn_norm.assign(w->ffn_norm[l], w->ffn_norm[l] + hidden);
    const orc_tensor* p = w->projections + l * 7;
    L.wq.load(p[0]);
    L.wk.load(p[1]);
    L.wv.load(p[2]);
    L.wo.load(p[3]);
    L.w1.load(p[4]);
    L.w2.load(p[5]);
    L.w3.load(p[6]);
  }
  m->lm_head.load(w->lm_head);
  return m.release();
}

void orc_model_destroy(orc_model* m) { delete m; }

size_t orc_model_weight_bytes(const orc_model* m) {  // src/model.rs:587-603
  size_t total = 0;
  for (const Layer& l : m->layers)
    for (const Linear* p : {&l.wq, &l.wk, &l.wv, &l.wo, &l.w1, &l.w2, &l.w3}) total += p->weight_bytes();
  return total + m->lm_head.weight_bytes();
}

int orc_model_forward(orc_model* m, uint32_t token, size_t pos, const int32_t* table, size_t table_len,
                      float* kv_cache, size_t kv_len, size_t block_size, float* logits) {
  std::vector<float> x;
  run_layers(*m, token, pos, Entry{table, table_len, 0, 0}, kv_cache, kv_len, block_size, x);
  m->lm_head.apply_parallel(logits, x.data());
  return 0;
}

int orc_model_prefill(orc_model* m, const uint32_t* tokens, size_t n, size_t start_pos, const int32_t* table,
                      size_t table_len, float* kv_cache, size_t kv_len, size_t block_size, float* logits) {
  if (n == 0) return -1;
  std::vector<float> x;
  for (size_t i = 0; i < n; ++i)
    run_layers(*m, tokens[i], start_pos + i, Entry{table, table_len, 0, 0}, kv_cache, kv_len, block_size, x);
  m->lm_head.apply_parallel(logits, x.data());
  return 0;
}

int orc_model_decode_batch(orc_model* m, const uint32_t* tokens, const int64_t* positions, const int32_t* tables,
                           size_t max_blocks, const int32_t* table_lens, size_t batch, float* kv_cache,
                           size_t kv_len, size_t block_size, float* logits) {
  if (batch == 0) return -1;
  std::vector<Entry> entries(batch);
  std::vector<size_t> pos(batch);
  for (size_t b = 0; b < batch; ++b) {
    entries[b] = Entry{tables + b * max_blocks, (size_t)table_lens[b], 0, 0};
    pos[b] = (size_t)positions[b];
  }
  std::vector<float> x;
  run_layers_batch(*m, tokens, pos.data(), entries, batch, kv_cache, kv_len, block_size, x);
  std::vector<float> stage(batch * m->lm_head.rows);
  m->lm_head.apply_batched(logits, x.data(), batch, stage.data());
  return 0;
}

int orc_model_prefill_batched(orc_model* m, const uint32_t* tokens, size_t n, size_t start_pos,
                              const int32_t* table, size_t table_len, float* kv_cache, size_t kv_len,
                              size_t block_size, size_t chunk_size, size_t capacity, float* logits) {
  if (n == 0) return -1;
  const size_t hidden = (size_t)m->cfg.hidden_size;
  chunk_size = std::min(std::max<size_t>(chunk_size, 1), std::max<size_t>(capacity, 1));
  std::vector<float> x;
  size_t last_hidden_at = 0;
  for (size_t c0 = 0; c0 < n; c0 += chunk_size) {
    const size_t len = std::min(chunk_size, n - c0);
    std::vector<size_t> pos(len);
    std::vector<Entry> entries(len, Entry{table, table_len, 0, 0});
    for (size_t i = 0; i < len; ++i) pos[i] = start_pos + c0 + i;
    run_layers_batch(*m, tokens + c0, pos.data(), entries, len, kv_cache, kv_len, block_size, x);
    last_hidden_at = len - 1;
  }
  m->lm_head.apply_parallel(logits, &x[last_hidden_at * hidden]);
  return 0;
}

}  // extern "C"
