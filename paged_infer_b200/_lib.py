"""ctypes binding of ``libpaged_infer_cuda.so`` (declarations follow
``include/paged_infer_cuda.h`` one to one).

There is no CPU fallback: if the shared library is missing, or no B200 is
visible when a context is created, the calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpaged_infer_cuda.so")

PI_OK = 0
PI_ERR_INVALID_ARG = -1
PI_ERR_OOM = -2
PI_ERR_CUDA = -3
PI_ERR_NCCL = -4
PI_ERR_TIMEOUT = -5
PI_ERR_UNSUPPORTED = -6

PI_SPLIT_NONE, PI_SPLIT_COLUMN, PI_SPLIT_ROW = 0, 1, 2
PI_F32, PI_INT8, PI_BF16 = 0, 1, 2
PROF_CLASSES = ("gemv", "gemm_tc", "attention", "rope_kv", "other", "collective")
PI_OPT_TENSOR_GEMM, PI_OPT_CUDA_GRAPH, PI_OPT_PDL, PI_OPT_GEMV_MAX_M, PI_OPT_ATTN_TMA, PI_OPT_FUSE_PLANES, PI_OPT_ATTN_SHARED = 1, 2, 3, 4, 5, 6, 7
PI_OPT_PEER_SPIN_LIMIT = 8
PI_OPT_TP_PUSH = 9
PI_OPT_ATTN_FLAT = 10


class PiError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"paged_infer_cuda error {status}: {message}")
        self.status = status
        self.message = message


class KvLayoutC(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("num_layers", "num_blocks", "block_size", "num_kv_heads", "head_dim")]


class ModelConfigC(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_int32), ("num_hidden_layers", C.c_int32), ("num_attention_heads", C.c_int32),
        ("num_key_value_heads", C.c_int32), ("intermediate_size", C.c_int32), ("vocab_size", C.c_int32),
        ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float), ("attention_window", C.c_int32),
        ("rope_style", C.c_int32), ("max_batch", C.c_int32), ("max_positions", C.c_int32),
    ]


class TensorC(C.Structure):
    _fields_ = [("kind", C.c_int32), ("quantize_on_load", C.c_int32), ("rows", C.c_int64), ("cols", C.c_int64),
                ("data", C.c_void_p), ("scales", C.c_void_p)]


class ModelWeightsC(C.Structure):
    _fields_ = [("token_embeddings_bf16", C.c_void_p), ("final_norm", C.c_void_p),
                ("attention_norm", C.POINTER(C.c_void_p)), ("ffn_norm", C.POINTER(C.c_void_p)),
                ("projections", C.POINTER(TensorC)), ("lm_head", TensorC)]


_P = C.c_void_p
_SZ = C.c_size_t
_I = C.c_int
_PP = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); must list every function the header declares.
SIGNATURES = {
    "pi_version": (C.c_char_p, []),
    "pi_last_error": (C.c_char_p, [_P]),
    "pi_ctx_create": (_I, [_I, _P, _PP]),
    "pi_nccl_unique_id": (_I, [_P]),
    "pi_ctx_create_tp": (_I, [_I, _P, _I, _I, _P, _PP]),
    "pi_tp_peer_export": (_I, [_P, _SZ, _P]),
    "pi_tp_peer_import": (_I, [_P, _P]),
    "pi_tp_peer_base": (_P, [_P]),
    "pi_tp_peer_import_pointers": (_I, [_P, _PP]),
    "pi_tp_exchange_add": (_I, [_P, _P, _P, _I, _I]),
    "pi_ctx_destroy": (None, [_P]),
    "pi_ctx_synchronize": (_I, [_P]),
    "pi_ctx_kernel_launches": (C.c_uint64, [_P]),
    "pi_ctx_reset_kernel_launches": (None, [_P]),
    "pi_ctx_set_option": (_I, [_P, _I, _I]),
    "pi_ctx_profile_begin": (_I, [_P]),
    "pi_ctx_profile_end": (_I, [_P, _P, _P]),
    "pi_quantize_rows_i8": (_I, [_P, _P, _SZ, _SZ, _P, _P]),
    "pi_quantize_rows_i8_dev": (_I, [_P, _P, _SZ, _SZ, _P, _P]),
    "pi_linear_create_i8": (_I, [_P, _SZ, _SZ, _P, _P, _I, _PP]),
    "pi_linear_create_quantized": (_I, [_P, _SZ, _SZ, _P, _I, _PP]),
    "pi_linear_create_bf16": (_I, [_P, _SZ, _SZ, _P, _I, _PP]),
    "pi_linear_create_f32": (_I, [_P, _SZ, _SZ, _P, _I, _PP]),
    "pi_linear_destroy": (None, [_P]),
    "pi_linear_rows": (_SZ, [_P]),
    "pi_linear_cols": (_SZ, [_P]),
    "pi_linear_weight_bytes": (_SZ, [_P]),
    "pi_linear_kind": (_I, [_P]),
    "pi_linear_read_i8": (_I, [_P, _P, _P, _P]),
    "pi_linear_apply": (_I, [_P, _P, _P, _P, _I]),
    "pi_linear_apply_host": (_I, [_P, _P, _P, _P, _I]),
    "pi_linear_apply_noalloc": (_I, [_P, _P, _P, _P, _I]),
    "pi_kv_pool_create": (_I, [_P, C.POINTER(KvLayoutC), _PP]),
    "pi_kv_pool_destroy": (None, [_P]),
    "pi_kv_pool_bytes": (_SZ, [_P]),
    "pi_kv_copy_block": (_I, [_P, _P, C.c_int32, C.c_int32]),
    "pi_kv_upload": (_I, [_P, _P, _P]),
    "pi_kv_download": (_I, [_P, _P, _P]),
    "pi_kv_write_token": (_I, [_P, _P, _I, C.c_int32, _I, _P, _P]),
    "pi_kv_read_token": (_I, [_P, _P, _I, C.c_int32, _I, _P, _P]),
    "pi_paged_attention": (_I, [_P, _P, _I, _I, _P, _SZ, _P, _SZ, _P, _I, _P, _P, _P, _I]),
    "pi_paged_attention_host": (_I, [_P, _P, _I, _I, _P, _P, _P, _I, _P, _P, _P, _I]),
    "pi_rms_norm_host": (_I, [_P, _P, _P, _I, _I, C.c_float]),
    "pi_rope_host": (_I, [_P, _P, _P, _I, _I, _I, C.c_float, _I]),
    "pi_swiglu_host": (_I, [_P, _P, _P, _SZ]),
    "pi_argmax_host": (_I, [_P, _P, _I, _I, _P]),
    "pi_model_create": (_I, [_P, C.POINTER(ModelConfigC), C.POINTER(ModelWeightsC), _PP]),
    "pi_model_create_synthetic": (_I, [_P, C.POINTER(ModelConfigC), C.c_uint64, C.c_float, _I, _I, _PP]),
    "pi_model_destroy": (None, [_P]),
    "pi_model_weight_bytes": (_SZ, [_P]),
    "pi_model_max_batch": (_I, [_P]),
    "pi_model_decode_batch_rows": (_I, [_P, _P, _P, _P, _P, _P, _I, _P, _I, _P, _I, _P, _P]),
    "pi_model_decode_batch": (_I, [_P, _P, _P, _P, _P, _P, _I, _P, _I, _P, _P]),
    "pi_model_prefill": (_I, [_P, _P, _P, _P, _I, _I, _P, _I, _I, _P, _P]),
    "pi_model_decode_multi": (_I, [_P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _P]),
    "pi_kv_fill_normal": (_I, [_P, _P, C.c_uint64, C.c_float]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the CUDA library; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m paged_infer_b200.build` "
                "(there is no CPU fallback for this path)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int, ctx=None) -> None:
    if status != PI_OK:
        msg = lib().pi_last_error(ctx)
        raise PiError(status, msg.decode() if msg else "")
