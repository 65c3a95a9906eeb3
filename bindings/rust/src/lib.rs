//! Bindings of `libpaged_infer_cuda.so` for the Paged-Infer engine: `ffi` is generated from
//! `include/paged_infer_cuda.h`; `cuda_backend` wraps it in the shapes the engine's call sites use.
pub mod cuda_backend;
pub mod ffi;
