// cuda_backend.rs - the Rust side of the device library: safe wrappers over `ffi.rs` that the engine calls where
// it calls the CPU kernels today.  Method names and argument meaning follow the reference's own
// (`LlamaWeights::decode_batch_into`, `prefill_batched`, `KvLayout::copy_block`), so the call sites change by a line
// or two each (listed in INTEGRATION.md, section 3).
//
// Not compiled in this repository's environment (no cargo / rustc): shipped as source, checked by reading only.
//
//   Engine::new                 ->  CudaBackend::new(device)  +  CudaLlama::from_weights  +  DeviceKvCache::new
//   weights.decode_batch_into   ->  CudaLlama::decode_batch_into    (greedy ids for all rows, logits for chosen rows)
//   weights.prefill_batched     ->  CudaLlama::prefill_batched
//   layout.copy_block           ->  DeviceKvCache::copy_block       (called from KvCacheManager::ensure_writable)
//
// Errors: the reference panics on shape mismatches; here every call returns `Result<_, CudaError>` carrying the
// library's message, so the engine can turn a refused batch into a failed request instead of a dead server.
#![allow(dead_code)]

use crate::ffi;
use std::ffi::CStr;
use std::ptr;

/// Status code + message of a failed library call.
#[derive(Debug, Clone)]
pub struct CudaError {
    pub status: i32,
    pub message: String,
}

impl std::fmt::Display for CudaError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "paged_infer_cuda error {}: {}", self.status, self.message)
    }
}
impl std::error::Error for CudaError {}

fn check(status: i32, ctx: *const ffi::PiCtx) -> Result<(), CudaError> {
    if status == ffi::PI_OK {
        return Ok(());
    }
    // SAFETY: pi_last_error never returns NULL and the string lives until the next call on the context.
    let message = unsafe { CStr::from_ptr(ffi::pi_last_error(ctx)) }.to_string_lossy().into_owned();
    Err(CudaError { status, message })
}

/// One device, one stream, one host thread - the engine is single-threaded, so this is `!Sync` on purpose.
pub struct CudaBackend {
    ctx: *mut ffi::PiCtx,
}

impl CudaBackend {
    pub fn new(device: i32) -> Result<Self, CudaError> {
        let mut ctx = ptr::null_mut();
        // SAFETY: plain out-pointer call; a NULL stream lets the library create its own.
        check(unsafe { ffi::pi_ctx_create(device, ptr::null_mut(), &mut ctx) }, ptr::null())?;
        Ok(Self { ctx })
    }

    /// Rank `rank` of `tp` processes on the GPUs of one node; `nccl_id` is rank 0's `pi_nccl_unique_id`.
    pub fn new_tensor_parallel(device: i32, rank: i32, tp: i32, nccl_id: &[u8; 128]) -> Result<Self, CudaError> {
        let mut ctx = ptr::null_mut();
        // SAFETY: the id is 128 readable bytes, as the library requires.
        check(
            unsafe { ffi::pi_ctx_create_tp(device, ptr::null_mut(), rank, tp, nccl_id.as_ptr().cast(), &mut ctx) },
            ptr::null(),
        )?;
        Ok(Self { ctx })
    }

    pub fn synchronize(&self) -> Result<(), CudaError> {
        check(unsafe { ffi::pi_ctx_synchronize(self.ctx) }, self.ctx)
    }
}

impl Drop for CudaBackend {
    fn drop(&mut self) {
        unsafe { ffi::pi_ctx_destroy(self.ctx) }
    }
}

/// The engine's `kv_cache: Vec<f32>` (src/engine.rs:206-207), resident in device memory.
pub struct DeviceKvCache<'b> {
    backend: &'b CudaBackend,
    pool: *mut ffi::PiKvPool,
    pub layout: ffi::PiKvLayout,
}

impl<'b> DeviceKvCache<'b> {
    /// `KvLayout` fields as `config.kv_layout(total_blocks, block_size)` gives them (src/model.rs:122-137); on a
    /// tensor-parallel backend pass this rank's share of the KV heads.
    pub fn new(backend: &'b CudaBackend, num_layers: usize, num_blocks: usize, block_size: usize, num_kv_heads: usize,
               head_dim: usize) -> Result<Self, CudaError> {
        let layout = ffi::PiKvLayout {
            num_layers: num_layers as i32,
            num_blocks: num_blocks as i32,
            block_size: block_size as i32,
            num_kv_heads: num_kv_heads as i32,
            head_dim: head_dim as i32,
        };
        let mut pool = ptr::null_mut();
        check(unsafe { ffi::pi_kv_pool_create(backend.ctx, &layout, &mut pool) }, backend.ctx)?;
        Ok(Self { backend, pool, layout })
    }

    /// `KvLayout::copy_block` (src/memory/layout.rs:82-96): duplicate one physical block across all layers.
    /// Stream-ordered: it runs before the forward pass that is queued next.  `KvCacheManager::ensure_writable`
    /// calls this where it called `layout.copy_block(kv_cache, slot.block, fresh)`.
    pub fn copy_block(&mut self, src: usize, dst: usize) -> Result<(), CudaError> {
        check(unsafe { ffi::pi_kv_copy_block(self.backend.ctx, self.pool, src as i32, dst as i32) }, self.backend.ctx)
    }

    /// Move an existing host cache (the reference's layout) onto the device, e.g. when migrating a warm engine.
    pub fn upload(&mut self, cache: &[f32]) -> Result<(), CudaError> {
        let l = &self.layout;
        let floats = l.num_layers as usize * l.num_blocks as usize * l.block_size as usize * l.num_kv_heads as usize * 2
            * l.head_dim as usize;
        assert_eq!(cache.len(), floats, "host cache does not match the layout");
        check(unsafe { ffi::pi_kv_upload(self.backend.ctx, self.pool, cache.as_ptr()) }, self.backend.ctx)
    }
}

impl Drop for DeviceKvCache<'_> {
    fn drop(&mut self) {
        unsafe { ffi::pi_kv_pool_destroy(self.pool) }
    }
}

/// One projection as the loader hands it over: int8 codes + scales (QUANT=int8), or bf16 checkpoint bits.
pub enum HostProjection<'w> {
    Int8 { rows: usize, cols: usize, codes: &'w [i8], scales: &'w [f32] },
    Bf16 { rows: usize, cols: usize, bits: &'w [u16] },
}

impl HostProjection<'_> {
    fn as_tensor(&self) -> ffi::PiTensor {
        match self {
            HostProjection::Int8 { rows, cols, codes, scales } => {
                assert_eq!(codes.len(), rows * cols);
                assert_eq!(scales.len(), *rows);
                ffi::PiTensor { kind: ffi::PI_INT8, quantize_on_load: 0, rows: *rows as i64, cols: *cols as i64,
                                data: codes.as_ptr().cast(), scales: scales.as_ptr() }
            }
            HostProjection::Bf16 { rows, cols, bits } => {
                assert_eq!(bits.len(), rows * cols);
                ffi::PiTensor { kind: ffi::PI_BF16, quantize_on_load: 0, rows: *rows as i64, cols: *cols as i64,
                                data: bits.as_ptr().cast(), scales: ptr::null() }
            }
        }
    }
}

/// `LlamaWeights` on the device.  Built once from the loaded host weights; the host copies can be dropped afterwards.
pub struct CudaLlama<'b> {
    backend: &'b CudaBackend,
    model: *mut ffi::PiModel,
    pub vocab_size: usize,
    pub max_batch: usize,
}

pub struct HostWeights<'w> {
    pub token_embeddings_bf16: &'w [u16],
    pub final_norm: &'w [f32],
    pub attention_norm: Vec<&'w [f32]>,
    pub ffn_norm: Vec<&'w [f32]>,
    /// per layer: wq, wk, wv, wo, w1 (gate), w2 (down), w3 (up)
    pub projections: Vec<[HostProjection<'w>; 7]>,
    pub lm_head: HostProjection<'w>,
}

impl<'b> CudaLlama<'b> {
    pub fn from_weights(backend: &'b CudaBackend, cfg: ffi::PiModelConfig, w: &HostWeights<'_>) -> Result<Self, CudaError> {
        let attn: Vec<*const f32> = w.attention_norm.iter().map(|s| s.as_ptr()).collect();
        let ffn: Vec<*const f32> = w.ffn_norm.iter().map(|s| s.as_ptr()).collect();
        let tensors: Vec<ffi::PiTensor> = w.projections.iter().flat_map(|l| l.iter().map(|p| p.as_tensor())).collect();
        let weights = ffi::PiModelWeights {
            token_embeddings_bf16: w.token_embeddings_bf16.as_ptr(),
            final_norm: w.final_norm.as_ptr(),
            attention_norm: attn.as_ptr(),
            ffn_norm: ffn.as_ptr(),
            projections: tensors.as_ptr(),
            lm_head: w.lm_head.as_tensor(),
        };
        let mut model = ptr::null_mut();
        // SAFETY: every pointer above outlives the call; the library copies what it keeps.
        check(unsafe { ffi::pi_model_create(backend.ctx, &cfg, &weights, &mut model) }, backend.ctx)?;
        Ok(Self { backend, model, vocab_size: cfg.vocab_size as usize, max_batch: cfg.max_batch as usize })
    }

    /// `decode_batch_into` (src/model.rs:1184-1207) for the engine's `run_groups` (src/engine.rs:702-760).
    /// `tables[b]` are the physical block ids of entry b's `BlockTable` (`slot.block.index`).  Returns the greedy
    /// token of every row; `logits_out` receives the full logits of `logit_rows` only (the sequences that sample
    /// with a temperature), `logit_rows.len() * vocab_size` floats.
    pub fn decode_batch_into(&self, tokens: &[u32], positions: &[usize], tables: &[&[i32]], kv: &mut DeviceKvCache<'_>,
                             logit_rows: &[usize], logits_out: &mut [f32]) -> Result<Vec<u32>, CudaError> {
        let b = tokens.len();
        assert!(b > 0 && positions.len() == b && tables.len() == b);
        assert!(logits_out.len() >= logit_rows.len() * self.vocab_size);
        let max_blocks = tables.iter().map(|t| t.len()).max().unwrap_or(0).max(1);
        let mut flat = vec![-1i32; b * max_blocks];
        let mut lens = vec![0i32; b];
        for (i, t) in tables.iter().enumerate() {
            flat[i * max_blocks..i * max_blocks + t.len()].copy_from_slice(t);
            lens[i] = t.len() as i32;
        }
        let pos: Vec<i32> = positions.iter().map(|&p| p as i32).collect();
        let rows: Vec<i32> = logit_rows.iter().map(|&r| r as i32).collect();
        let mut ids = vec![0u32; b];
        check(
            unsafe {
                ffi::pi_model_decode_batch_rows(self.backend.ctx, self.model, kv.pool, tokens.as_ptr(), pos.as_ptr(), flat.as_ptr(),
                                                max_blocks as i32, lens.as_ptr(), b as i32,
                                                if rows.is_empty() { ptr::null() } else { rows.as_ptr() }, rows.len() as i32,
                                                if rows.is_empty() { ptr::null_mut() } else { logits_out.as_mut_ptr() },
                                                ids.as_mut_ptr())
            },
            self.backend.ctx,
        )?;
        Ok(ids)
    }

    /// `prefill_batched` (src/model.rs:1222-1255): logits of the last prompt position into `last_logits`
    /// (`vocab_size` floats), its greedy token as the return value.  `chunk_size` is clamped to `max_batch`.
    pub fn prefill_batched(&self, tokens: &[u32], start_pos: usize, table: &[i32], kv: &mut DeviceKvCache<'_>, chunk_size: usize,
                           last_logits: &mut [f32]) -> Result<u32, CudaError> {
        assert!(!tokens.is_empty(), "prefill needs at least one token");
        assert!(last_logits.len() >= self.vocab_size);
        let mut id = 0u32;
        check(
            unsafe {
                ffi::pi_model_prefill(self.backend.ctx, self.model, kv.pool, tokens.as_ptr(), tokens.len() as i32, start_pos as i32,
                                      table.as_ptr(), table.len() as i32, chunk_size as i32, last_logits.as_mut_ptr(), &mut id)
            },
            self.backend.ctx,
        )?;
        Ok(id)
    }
}

impl Drop for CudaLlama<'_> {
    fn drop(&mut self) {
        unsafe { ffi::pi_model_destroy(self.model) }
    }
}
