"""paged_infer_b200: the int8 decode hot path of Paged-Infer on B200 (sm_100a).

The product is ``libpaged_infer_cuda.so`` (C ABI in ``include/paged_infer_cuda.h``);
this package is the thin host side above it: a ctypes binding (``_lib``), the
mirror of the reference's Rust interface (``api``) and the checkpoint reader
(``loader``).  Importing the package does not load the CUDA library; the first
call that needs it does, and raises if it was not built.
"""
from .loader import (QUANT_F32, QUANT_INT8, ROPE_INTERLEAVED, ROPE_NEOX, HostWeights, LlamaConfig, bf16_bits_to_f32,
                     f32_to_bf16_bits, load_weights, read_safetensors)

__all__ = ["QUANT_F32", "QUANT_INT8", "ROPE_INTERLEAVED", "ROPE_NEOX", "HostWeights", "LlamaConfig", "bf16_bits_to_f32",
           "f32_to_bf16_bits", "load_weights", "read_safetensors", "api", "build"]
