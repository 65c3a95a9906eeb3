/*
 * paged_infer_cuda.h - C ABI of libpaged_infer_cuda.so
 *
 * A B200 (sm_100a) implementation of the quantised decode hot path of
 * Paged-Infer: per-row int8 weight-only projections, their quantiser, the
 * paged-attention read over the engine's block tables, and the per-token glue
 * between them, with the physical KV pool resident in device memory.
 *
 * The reference (a Rust crate) has no FFI of its own for this path; the seam is
 * the set of Rust methods cited beside each entry point below ("replaces ...",
 * paths relative to the reference checkout).  A Rust `extern "C"` block can bind
 * these declarations verbatim.
 *
 * Conventions
 *  - Every call returns a pi_status; nothing aborts or throws across the ABI.
 *    The reference's assert!/panic conditions become PI_ERR_INVALID_ARG.
 *    pi_last_error() returns a description of the last failure on that context.
 *  - One pi_ctx = one host thread = one CUDA stream (the reference engine is
 *    single-threaded by construction, src/bin/http_server.rs:143-266).
 *  - "_host" pointers are host memory borrowed for the duration of the call.
 *    "_dev" pointers are device memory on the context's device.  Handles own
 *    their device memory.
 *  - Calls that write to a host output pointer have completed when they return;
 *    calls that only touch device memory are ordered on the context's stream.
 *  - Matrices are row-major [out_features][in_features] (y = x * W^T), as in the
 *    reference (src/model.rs:140-199).
 *  - The device layout of weights and of the KV pool is private to the library.
 */
#ifndef PAGED_INFER_CUDA_H
#define PAGED_INFER_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t pi_status;
enum {
  PI_OK = 0,
  PI_ERR_INVALID_ARG = -1,
  PI_ERR_OOM = -2,
  PI_ERR_CUDA = -3,
  PI_ERR_NCCL = -4,
  PI_ERR_TIMEOUT = -5,
  PI_ERR_UNSUPPORTED = -6
};

typedef struct pi_ctx pi_ctx;
typedef struct pi_linear pi_linear;
typedef struct pi_kv_pool pi_kv_pool;
typedef struct pi_model pi_model;

/* ---- context --------------------------------------------------------------- */

/* Library version string, e.g. "paged_infer_cuda 0.1 (sm_100a)". */
const char* pi_version(void);

/* Message for the last error on `ctx`; with ctx == NULL, for the last failed
 * pi_ctx_create* on this thread.  Never NULL. */
const char* pi_last_error(const pi_ctx* ctx);

/* Create a context on CUDA device `device`.  `stream` is a cudaStream_t the
 * caller owns, or NULL to let the context create its own.
 * Replaces: nothing in the reference (its kernels run on the calling thread);
 * it takes the place of the rayon pool + GpuContext::new (src/gpu.rs:18-60). */
pi_status pi_ctx_create(int device, void* stream, pi_ctx** out);

/* Tensor-parallel context: rank `rank` of `tp` (1, 2, 4 or 8) processes, one
 * per GPU of one node.  `nccl_unique_id` is the 128-byte id produced by
 * pi_nccl_unique_id() on rank 0 and distributed by the host (any transport).
 * Column-split projections keep rows [rank*rows/tp, (rank+1)*rows/tp); row-split
 * projections keep the matching column slice and are followed by one
 * all-reduce.  No counterpart in the reference (it has no multi-device code). */
pi_status pi_nccl_unique_id(void* out_128_bytes);
/* nccl_unique_id may be NULL: the context then has no NCCL communicator and only the peer-memory exchange below
 * works (the vocab-split LM head's all-gather, which needs NCCL, fails with PI_ERR_NCCL). */
pi_status pi_ctx_create_tp(int device, void* stream, int rank, int tp,
                           const void* nccl_unique_id, pi_ctx** out);
/* Optional peer-memory path for the exchange after the row-split projections (o, down): instead of an NCCL
 * all-reduce, one kernel per exchange reads every peer's partial sums straight out of that peer's memory (NVLink
 * P2P loads), adds them in rank order and folds in the residual add.  Set-up: every rank calls
 * pi_tp_peer_export(ctx, max_rows * hidden_size, handle) -> 64 bytes, the host gathers the tp handles in rank order
 * (any transport) and every rank calls pi_tp_peer_import(ctx, all_handles).  Without it the NCCL path is used.
 * Ranks must be processes on the GPUs of one node with peer access.  Waits on a peer are bounded: a rank whose
 * peer never arrives reports PI_ERR_TIMEOUT at the next synchronising call.  No counterpart in the reference. */
#define PI_TP_PEER_HANDLE_BYTES 64
pi_status pi_tp_peer_export(pi_ctx* ctx, size_t max_floats, void* handle_out_64_bytes);
pi_status pi_tp_peer_import(pi_ctx* ctx, const void* handles_tp_times_64_bytes);
/* The same set-up for a host that drives all GPUs from ONE process (the reference engine is a single process,
 * src/bin/http_server.rs:143-266): a process cannot open IPC handles of its own allocations, so it passes the base
 * pointer of every rank's buffer instead (pi_tp_peer_base of that rank's context after pi_tp_peer_export, in rank
 * order; the host has enabled peer access between the devices).  No counterpart in the reference. */
void* pi_tp_peer_base(const pi_ctx* ctx);
pi_status pi_tp_peer_import_pointers(pi_ctx* ctx, void* const* bases_tp);
/* The exchange on its own: x_dev[rows x cols] += sum over all ranks of partial_dev[rows x cols] (the partial sums of
 * a row-split projection), added in rank order so that every rank ends with the same bits.  Peer-memory path when
 * it is set up, NCCL all-reduce otherwise.  Every rank must call it with the same shape.  After a
 * PI_ERR_TIMEOUT the ranks' slots are out of step: the peer path is disabled for the context and later
 * exchanges use NCCL.  Ranks must enter each exchange within the wait budget of their peers (about a second by
 * default, PI_OPT_PEER_SPIN_LIMIT) and must synchronise on the host (a barrier) before any of them destroys its
 * context, because peers read its buffer directly.  No counterpart in the reference. */
pi_status pi_tp_exchange_add(pi_ctx* ctx, const float* partial_dev, float* x_dev, int rows, int cols);
void pi_ctx_destroy(pi_ctx* ctx);
/* Block until everything queued on the context's stream has finished. */
pi_status pi_ctx_synchronize(pi_ctx* ctx);
/* Kernels launched by this context since creation (or since the last reset). */
uint64_t pi_ctx_kernel_launches(const pi_ctx* ctx);
void pi_ctx_reset_kernel_launches(pi_ctx* ctx);
/* Per-kernel-class device timing.  Between begin and end every launch of the
 * context is bracketed by CUDA events on its stream (which serialises
 * launches that would otherwise overlap); end waits for the stream and returns,
 * per class, the summed device time in milliseconds and the number of launches.
 * Classes: */
enum { PI_PROF_GEMV = 0, PI_PROF_GEMM_TC = 1, PI_PROF_ATTENTION = 2, PI_PROF_ROPE_KV = 3, PI_PROF_OTHER = 4,
       PI_PROF_COLLECTIVE = 5, PI_PROF_CLASSES = 6 };
pi_status pi_ctx_profile_begin(pi_ctx* ctx);
pi_status pi_ctx_profile_end(pi_ctx* ctx, double* ms_out /*[PI_PROF_CLASSES]*/, uint64_t* launches_out /*[PI_PROF_CLASSES]*/);
/* Tuning knobs (the 0/1 ones default on). */
enum { PI_OPT_TENSOR_GEMM = 1, PI_OPT_CUDA_GRAPH = 2, PI_OPT_PDL = 3, PI_OPT_GEMV_MAX_M = 4, PI_OPT_ATTN_TMA = 5, PI_OPT_FUSE_PLANES = 6, PI_OPT_ATTN_SHARED = 7,
       PI_OPT_PEER_SPIN_LIMIT = 8 /* polls, 64 ns apart, that a rank waits for a peer's partial sums; 0 = default */,
       PI_OPT_TP_PUSH = 9 /* peer path: row-split projections store their partial sums into every rank's buffer themselves */,
       PI_OPT_ATTN_FLAT = 10 /* batched decode attention over one flat tile list cut into equal ranges per resident warp:
                                0 never, 1 (default) inside a model forward, 2 also for a single pi_paged_attention call */ };
pi_status pi_ctx_set_option(pi_ctx* ctx, int option, int value);

/* ---- quantiser --------------------------------------------------------------- */

/* Per-row symmetric absmax int8: scale[r] = max|w[r,:]| / 127 (1.0 for an
 * all-zero row), code = round_half_away(w / scale) clamped to +-127.  Bit-exact
 * with the reference.  Replaces: math::quantize_rows_i8 (src/math.rs:456-469). */
pi_status pi_quantize_rows_i8(pi_ctx* ctx, const float* w_host, size_t rows, size_t cols,
                              int8_t* q_host_out, float* scales_host_out);
/* Same, device to device (row stride = cols). */
pi_status pi_quantize_rows_i8_dev(pi_ctx* ctx, const float* w_dev, size_t rows, size_t cols,
                                  int8_t* q_dev_out, float* scales_dev_out);

/* ---- projections ------------------------------------------------------------- */

typedef enum { PI_SPLIT_NONE = 0, PI_SPLIT_COLUMN = 1, PI_SPLIT_ROW = 2 } pi_split;
enum { PI_F32 = 0, PI_INT8 = 1, PI_BF16 = 2 };

/* Replaces: QuantizedLinear {rows, cols, weight, scales} (src/model.rs:164-199).
 * The codes and scales are copied to the device (sharded per `split` on a
 * tensor-parallel context; scales of a row-split matrix stay whole-row). */
pi_status pi_linear_create_i8(pi_ctx* ctx, size_t rows, size_t cols, const int8_t* q_host,
                              const float* scales_host, pi_split split, pi_linear** out);
/* Replaces: QuantizedLinear::from_packed (src/model.rs:173-182): quantise f32
 * weights on the device and keep the int8 form. */
pi_status pi_linear_create_quantized(pi_ctx* ctx, size_t rows, size_t cols, const float* w_host,
                                     pi_split split, pi_linear** out);
/* Replaces: PackedLinear (src/model.rs:140-162) for checkpoint weights, which
 * are bf16 on disk and widened exactly to f32 by the reference
 * (math::pack_bf16_to_f32, src/math.rs:66-71): kept as bf16, accumulated in f32. */
pi_status pi_linear_create_bf16(pi_ctx* ctx, size_t rows, size_t cols, const uint16_t* w_bf16_host,
                                pi_split split, pi_linear** out);
/* Replaces: PackedLinear holding arbitrary f32 weights. */
pi_status pi_linear_create_f32(pi_ctx* ctx, size_t rows, size_t cols, const float* w_host,
                               pi_split split, pi_linear** out);
void pi_linear_destroy(pi_linear* lin);
/* Replaces: Projection::rows/cols/weight_bytes (src/model.rs:261-280); rows and
 * cols are the full (unsharded) shape, bytes those held on this device. */
size_t pi_linear_rows(const pi_linear* lin);
size_t pi_linear_cols(const pi_linear* lin);
size_t pi_linear_weight_bytes(const pi_linear* lin);
int pi_linear_kind(const pi_linear* lin);
/* Copy this device's int8 codes [local_rows x local_cols] and scales back. */
pi_status pi_linear_read_i8(pi_ctx* ctx, const pi_linear* lin, int8_t* q_host_out, float* scales_host_out);

/* out[m][r] = scale[r] * sum_k W[r][k] * x[m][k], f32 accumulation.
 * x_dev is [M x cols], out_dev is [M x rows] (batch-major, like the
 * reference's apply_batched result after its transpose).
 * Replaces: Projection::apply_parallel (M == 1; math::matvec_i8_weight_parallel,
 * src/math.rs:473-512, and the f32 twin :93-129) and Projection::apply_batched
 * (src/model.rs:247-259; math::matmat_i8_weight_parallel, src/math.rs:223-275,
 * plus transpose_rb_to_br :281-290).  On a tensor-parallel context this applies
 * the local shard only (no all-reduce). */
pi_status pi_linear_apply(pi_ctx* ctx, const pi_linear* lin, const float* x_dev, float* out_dev, int M);
/* Same with host buffers: copies x in, runs, copies out back, synchronises. */
pi_status pi_linear_apply_host(pi_ctx* ctx, const pi_linear* lin, const float* x_host, float* out_host, int M);
/* pi_linear_apply for callers that must not allocate while they run it.  This
 * entry point has no counterpart in the reference.  The tensor-core projection
 * keeps three bf16 planes of the activations and one factor per activation row
 * in scratch memory; pi_linear_apply grows that scratch with cudaMalloc when a
 * larger shape arrives.  A caller that is inside a CUDA stream capture, that has
 * a latency budget a driver allocation would break, or that has given all
 * device memory to its own pool cannot afford that, so this variant uses a
 * fixed scratch area built into the library (about 3 MiB, held by every GPU
 * that loads the library until the process exits) and calls no cudaMalloc,
 * cudaFree or other allocating routine.
 *  - Limits: int8 projection with >= 32 rows and a multiple of 128 columns,
 *    columns <= 8192, 1 <= M <= 64.  Anything else returns PI_ERR_INVALID_ARG.
 *  - x_dev is [M x cols], out_dev is [M x rows], both dense, as in pi_linear_apply;
 *    the work is ordered on the context's stream.
 *  - The first call on a device looks up the scratch area's device address and
 *    sets a kernel attribute; make that first call before any stream capture.
 *  - The scratch area is shared by all calls on the device and keeps the last
 *    call's contents; nothing in it needs clearing, but two calls whose kernels
 *    overlap on the GPU (other streams or contexts) race on it: order them. */
pi_status pi_linear_apply_noalloc(pi_ctx* ctx, const pi_linear* lin, const float* x_dev, float* out_dev, int M);

/* ---- KV pool ------------------------------------------------------------------ */

/* Replaces: KvLayout (src/memory/layout.rs:18-41). */
typedef struct {
  int32_t num_layers, num_blocks, block_size, num_kv_heads, head_dim;
} pi_kv_layout;

/* Replaces: the engine's `kv_cache: Vec<f32>` (src/engine.rs:206-207), now in
 * device memory.  Contents start undefined, like a pool that is never read
 * before it is written. */
pi_status pi_kv_pool_create(pi_ctx* ctx, const pi_kv_layout* layout, pi_kv_pool** out);
void pi_kv_pool_destroy(pi_kv_pool* pool);
size_t pi_kv_pool_bytes(const pi_kv_pool* pool);
/* Replaces: KvLayout::copy_block (src/memory/layout.rs:82-96): duplicate one
 * physical block across all layers (copy-on-write).  src == dst is
 * PI_ERR_INVALID_ARG where the reference asserts. */
pi_status pi_kv_copy_block(pi_ctx* ctx, pi_kv_pool* pool, int32_t src, int32_t dst);
/* Whole-pool transfer in the REFERENCE's layout
 * [layer][block][token][kv_head][k|v][head_dim] (src/memory/layout.rs:56-71),
 * for tests and for migrating an existing host cache. */
pi_status pi_kv_upload(pi_ctx* ctx, pi_kv_pool* pool, const float* cache_host);
pi_status pi_kv_download(pi_ctx* ctx, const pi_kv_pool* pool, float* cache_host_out);
/* One token's K and V ([num_kv_heads x head_dim] each) of one layer. */
pi_status pi_kv_write_token(pi_ctx* ctx, pi_kv_pool* pool, int layer, int32_t block, int tok,
                            const float* k_host, const float* v_host);
pi_status pi_kv_read_token(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int32_t block, int tok,
                           float* k_host_out, float* v_host_out);

/* ---- paged attention ---------------------------------------------------------- */

/* Entry b attends positions start[b] ..= pos[b] of the sequence whose logical
 * blocks are block_tables[b*max_blocks .. +table_lens[b]] (physical ids).
 * A position whose logical block index is >= table_lens[b] scores -inf and its
 * V is never read; an empty or fully masked window yields zeros.
 * q_dev/out_dev are [B][num_heads][head_dim] with row strides q_stride /
 * out_stride floats between entries.  Query head h reads KV head
 * h / (num_heads / num_kv_heads).
 * Replaces: PagedAttention::run + AttnEntry (src/attention.rs:58-265) and
 * BlockTable::get_physical_location (src/memory/block_table.rs:50-61). */
pi_status pi_paged_attention(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads,
                             const float* q_dev, size_t q_stride, float* out_dev, size_t out_stride,
                             const int32_t* block_tables_host, int max_blocks, const int32_t* table_lens_host,
                             const int32_t* pos_host, const int32_t* start_host, int B);
/* Same with host q/out ([B][num_heads][head_dim], dense). */
pi_status pi_paged_attention_host(pi_ctx* ctx, const pi_kv_pool* pool, int layer, int num_heads,
                                  const float* q_host, float* out_host,
                                  const int32_t* block_tables_host, int max_blocks, const int32_t* table_lens_host,
                                  const int32_t* pos_host, const int32_t* start_host, int B);

/* ---- per-token glue (device compute, host buffers; used by the unit tests) ---- */

/* x[r][:] = x[r][:] * rsqrt(mean(x^2) + eps) * weight.  Replaces math::rms_norm (src/math.rs:4-22). */
pi_status pi_rms_norm_host(pi_ctx* ctx, float* x_host_inout, const float* weight_host, int rows, int n, float eps);
/* Rotate `heads` vectors of length head_dim per row at position pos[r].
 * style 0 = NeoX pairs (j, j + head_dim/2), 1 = interleaved (2j, 2j+1).
 * Replaces math::rope_table + rope_rotate (src/math.rs:331-367). */
pi_status pi_rope_host(pi_ctx* ctx, float* x_host_inout, const int32_t* pos_host, int rows, int heads,
                       int head_dim, float theta, int style);
/* gate[i] = silu(gate[i]) * up[i].  Replaces math::swiglu (src/math.rs:292-302). */
pi_status pi_swiglu_host(pi_ctx* ctx, float* gate_host_inout, const float* up_host, size_t n);
/* Index of the maximum under IEEE total order; ties go to the LAST index.
 * Replaces sampling::argmax (src/sampling.rs:140-147). */
pi_status pi_argmax_host(pi_ctx* ctx, const float* logits_host, int rows, int n, uint32_t* out_host);

/* ---- model forward ------------------------------------------------------------- */

/* Replaces: LlamaConfig (src/model.rs:14-53). */
typedef struct {
  int32_t hidden_size, num_hidden_layers, num_attention_heads, num_key_value_heads;
  int32_t intermediate_size, vocab_size;
  float rms_norm_eps, rope_theta;
  int32_t attention_window; /* < 0: full causal attention (None) */
  int32_t rope_style;       /* 0 NeoX, 1 interleaved */
  int32_t max_batch;        /* BatchScratch capacity (src/model.rs:540-572) */
  int32_t max_positions;    /* longest sequence the rotary table is built for; grows on demand */
} pi_model_config;

typedef struct {
  int32_t kind;             /* PI_F32, PI_INT8 or PI_BF16 */
  int32_t quantize_on_load; /* f32/bf16 input: quantise to int8 on the device (Quantization::Int8) */
  int64_t rows, cols;
  const void* data;         /* host, row-major [rows][cols] */
  const float* scales;      /* host [rows], PI_INT8 only */
} pi_tensor;

/* Replaces: LlamaWeights as built by ModelLoader::load_weights (src/model.rs:380-446). */
typedef struct {
  const uint16_t* token_embeddings_bf16; /* [vocab][hidden] */
  const float* final_norm;               /* [hidden] */
  const float* const* attention_norm;    /* [layers] -> [hidden] */
  const float* const* ffn_norm;          /* [layers] -> [hidden] */
  const pi_tensor* projections;          /* [layers*7]: wq, wk, wv, wo, w1 (gate), w2 (down), w3 (up) */
  pi_tensor lm_head;
} pi_model_weights;

pi_status pi_model_create(pi_ctx* ctx, const pi_model_config* cfg, const pi_model_weights* weights, pi_model** out);
/* Random-init N(0, std) weights generated and quantised on the device (for
 * shapes too large to build on the host).  quant: PI_INT8 or PI_BF16;
 * lm_head_kind likewise.  No counterpart in the reference. */
pi_status pi_model_create_synthetic(pi_ctx* ctx, const pi_model_config* cfg, uint64_t seed, float std,
                                    int quant, int lm_head_kind, pi_model** out);
void pi_model_destroy(pi_model* model);
/* Replaces: LlamaWeights::weight_bytes (src/model.rs:587-603), bytes on this device. */
size_t pi_model_weight_bytes(const pi_model* model);
/* Rows one batched forward can take (the max_batch the model was created with).
 * Replaces: BatchScratch::capacity (src/model.rs:540-572). */
int pi_model_max_batch(const pi_model* model);

/* Advance B sequences by one token each.  tokens[b] lands at positions[b] of
 * the sequence with block table row b; its K/V are written to the pool (skipped
 * silently when that position's block is unmapped) before any attention of the
 * layer reads.  logits_host_or_null receives [B][vocab]; argmax_host_or_null
 * receives B greedy token ids (ties to the last index).  Either may be NULL.
 * Replaces: LlamaWeights::decode_batch_into (src/model.rs:1184-1207) and, for
 * B == 1, forward_into (:659-681). */
pi_status pi_model_decode_batch(pi_ctx* ctx, pi_model* model, pi_kv_pool* pool,
                                const uint32_t* tokens_host, const int32_t* positions_host,
                                const int32_t* block_tables_host, int max_blocks, const int32_t* table_lens_host,
                                int B, float* logits_host_or_null, uint32_t* argmax_host_or_null);

/* pi_model_decode_batch with the logits of SOME rows only: argmax_host receives all B greedy ids, and
 * logits_host receives n_logit_rows x vocab floats, row i being the logits of batch row logit_rows_host[i]
 * (for the sequences the host samples itself, temperature > 0; greedy ones need only their id).
 * Replaces: the per-sequence read of BatchScratch::logits_for_mut in Engine::run_groups (src/engine.rs:742-755). */
pi_status pi_model_decode_batch_rows(pi_ctx* ctx, pi_model* model, pi_kv_pool* pool,
                                     const uint32_t* tokens_host, const int32_t* positions_host,
                                     const int32_t* block_tables_host, int max_blocks, const int32_t* table_lens_host,
                                     int B, const int32_t* logit_rows_host, int n_logit_rows,
                                     float* logits_host, uint32_t* argmax_host);

/* Consume n prompt tokens of one sequence starting at start_pos, `chunk`
 * positions per pass, and return the logits of the last position only.
 * Replaces: LlamaWeights::prefill_batched (src/model.rs:1222-1255) and
 * prefill_into (:726-751, chunk == 1). */
pi_status pi_model_prefill(pi_ctx* ctx, pi_model* model, pi_kv_pool* pool, const uint32_t* tokens_host, int n,
                           int start_pos, const int32_t* block_table_host, int table_len, int chunk,
                           float* last_logits_host_or_null, uint32_t* argmax_host_or_null);

/* n_steps greedy decode steps of the same B sequences without returning to the
 * host in between: step s feeds the argmax of step s-1 at position
 * positions[b] + s.  The block tables must already map every position that
 * will be written (an unmapped position's K/V write is skipped, as always).
 * out_tokens_host receives [n_steps][B] token ids.
 * Replaces: n_steps iterations of Engine::step's decode phase for sequences
 * sampled greedily (src/engine.rs:602-761 with temperature 0), minus the host
 * bookkeeping between them. */
pi_status pi_model_decode_multi(pi_ctx* ctx, pi_model* model, pi_kv_pool* pool,
                                const uint32_t* tokens_host, const int32_t* positions_host,
                                const int32_t* block_tables_host, int max_blocks, const int32_t* table_lens_host,
                                int B, int n_steps, uint32_t* out_tokens_host);

/* Fill the whole pool with N(0, std) values (synthetic KV for benchmarks).
 * No counterpart in the reference. */
pi_status pi_kv_fill_normal(pi_ctx* ctx, pi_kv_pool* pool, uint64_t seed, float std);

#ifdef __cplusplus
}
#endif
#endif /* PAGED_INFER_CUDA_H */
