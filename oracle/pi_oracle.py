"""ctypes bindings for the CPU oracle (``libpi_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The
CUDA library and the ``paged_infer_b200`` package never import this module.

The oracle restates the reference's CPU path (Rust ``src/math.rs``,
``src/simd.rs``, ``src/attention.rs``, ``src/memory/layout.rs``,
``src/model.rs``); see ``pi_oracle.h`` for the file:line of each function.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libpi_oracle.so")

F32 = 0
INT8 = 1
BF16 = 2


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc, no CUDA)."""
    src = [os.path.join(_HERE, n) for n in ("pi_oracle.cpp", "pi_oracle.h", "Makefile")]
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src
    )
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "libpi_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


class KvLayout(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("num_layers", "num_blocks", "block_size", "num_kv_heads", "head_dim")]

    def total_floats(self) -> int:
        return self.num_layers * self.num_blocks * self.block_size * self.num_kv_heads * 2 * self.head_dim


class Tensor(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("rows", C.c_int64),
        ("cols", C.c_int64),
        ("data", C.c_void_p),
        ("scales", C.c_void_p),
    ]


class ModelConfig(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_int64),
        ("num_hidden_layers", C.c_int64),
        ("num_attention_heads", C.c_int64),
        ("num_key_value_heads", C.c_int64),
        ("intermediate_size", C.c_int64),
        ("vocab_size", C.c_int64),
        ("rms_norm_eps", C.c_float),
        ("rope_theta", C.c_float),
        ("attention_window", C.c_int64),
        ("rope_style", C.c_int32),
    ]


class ModelWeights(C.Structure):
    _fields_ = [
        ("token_embeddings_bf16", C.c_void_p),
        ("final_norm", C.c_void_p),
        ("attention_norm", C.POINTER(C.c_void_p)),
        ("ffn_norm", C.POINTER(C.c_void_p)),
        ("projections", C.POINTER(Tensor)),
        ("lm_head", Tensor),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(L: C.CDLL) -> None:
    sz, f, p, i = C.c_size_t, C.c_float, C.c_void_p, C.c_int
    L.orc_backend_avx2.restype = i
    L.orc_force_scalar.argtypes = [i]
    L.orc_num_threads.restype = i
    L.orc_set_num_threads.argtypes = [i]
    for name in ("orc_dot_naive", "orc_dot_scalar", "orc_dot_i8_scalar", "orc_dot", "orc_dot_i8"):
        fn = getattr(L, name)
        fn.argtypes = [p, p, sz]
        fn.restype = f
    L.orc_dot_multi.argtypes = [p, p, sz, sz, i, p]
    L.orc_dot_i8_multi.argtypes = [p, p, sz, sz, i, p]
    L.orc_axpy.argtypes = [p, f, p, sz]
    L.orc_quantize_rows_i8.argtypes = [p, sz, sz, p, p]
    L.orc_matvec_i8.argtypes = [p, p, p, p, sz, sz]
    L.orc_matvec_f32.argtypes = [p, p, p, sz, sz]
    L.orc_matvec_f32_sequential.argtypes = [p, p, p, sz, sz]
    L.orc_matmat_i8.argtypes = [p, p, p, p, sz, sz, sz, i]
    L.orc_matmat_f32.argtypes = [p, p, p, sz, sz, sz, i]
    L.orc_transpose_rb_to_br.argtypes = [p, p, sz, sz]
    L.orc_pack_bf16_to_f32.argtypes = [p, p, sz]
    L.orc_rms_norm.argtypes = [p, p, sz, f]
    L.orc_silu.argtypes = [f]
    L.orc_silu.restype = f
    L.orc_swiglu.argtypes = [p, p, sz]
    L.orc_rope_table.argtypes = [sz, sz, f, p, p]
    L.orc_rope_rotate.argtypes = [p, sz, p, p, i]
    L.orc_softmax_in_place.argtypes = [p, sz]
    L.orc_argmax.argtypes = [p, sz]
    L.orc_argmax.restype = sz
    L.orc_kv_total_floats.argtypes = [C.POINTER(KvLayout)]
    L.orc_kv_total_floats.restype = sz
    L.orc_kv_index.argtypes = [C.POINTER(KvLayout), sz, sz, sz, sz, i]
    L.orc_kv_index.restype = sz
    L.orc_kv_copy_block.argtypes = [C.POINTER(KvLayout), p, sz, sz]
    L.orc_kv_copy_block.restype = i
    L.orc_lane_width.argtypes = [sz] * 5
    L.orc_lane_width.restype = sz
    L.orc_paged_attention_run.argtypes = [p, p, p, p, C.POINTER(KvLayout), sz, sz, sz, sz, sz, sz, p, sz, p, p, p, sz, sz]
    L.orc_paged_attention_run.restype = i
    L.orc_model_create.argtypes = [C.POINTER(ModelConfig), C.POINTER(ModelWeights)]
    L.orc_model_create.restype = p
    L.orc_model_destroy.argtypes = [p]
    L.orc_model_weight_bytes.argtypes = [p]
    L.orc_model_weight_bytes.restype = sz
    L.orc_model_forward.argtypes = [p, C.c_uint32, sz, p, sz, p, sz, sz, p]
    L.orc_model_forward.restype = i
    L.orc_model_prefill.argtypes = [p, p, sz, sz, p, sz, p, sz, sz, p]
    L.orc_model_prefill.restype = i
    L.orc_model_decode_batch.argtypes = [p, p, p, p, sz, p, sz, p, sz, sz, p]
    L.orc_model_decode_batch.restype = i
    L.orc_model_prefill_batched.argtypes = [p, p, sz, sz, p, sz, p, sz, sz, sz, sz, p]
    L.orc_model_prefill_batched.restype = i


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- simd.rs ---------------------------------------------------------------
def backend() -> str:
    return "avx2+fma" if lib().orc_backend_avx2() else "scalar"


def num_threads() -> int:
    return lib().orc_num_threads()


def dot(a, b) -> float:
    a, b = _f32(a), _f32(b)
    return lib().orc_dot(_ptr(a), _ptr(b), min(a.size, b.size))


def dot_scalar(a, b) -> float:
    a, b = _f32(a), _f32(b)
    return lib().orc_dot_scalar(_ptr(a), _ptr(b), min(a.size, b.size))


def dot_i8(w, x) -> float:
    w = np.ascontiguousarray(w, dtype=np.int8)
    x = _f32(x)
    return lib().orc_dot_i8(_ptr(w), _ptr(x), min(w.size, x.size))


def dot_i8_scalar(w, x) -> float:
    w = np.ascontiguousarray(w, dtype=np.int8)
    x = _f32(x)
    return lib().orc_dot_i8_scalar(_ptr(w), _ptr(x), min(w.size, x.size))


def dot_multi(w, x_block, stride: int, bt: int) -> np.ndarray:
    w, x_block = _f32(w), _f32(x_block)
    out = np.zeros(bt, np.float32)
    lib().orc_dot_multi(_ptr(w), _ptr(x_block), w.size, stride, bt, _ptr(out))
    return out


def dot_i8_multi(w, x_block, stride: int, bt: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.int8)
    x_block = _f32(x_block)
    out = np.zeros(bt, np.float32)
    lib().orc_dot_i8_multi(_ptr(w), _ptr(x_block), w.size, stride, bt, _ptr(out))
    return out


def axpy(out: np.ndarray, weight: float, v) -> None:
    v = _f32(v)
    assert out.dtype == np.float32 and out.flags.c_contiguous
    lib().orc_axpy(_ptr(out), weight, _ptr(v), min(out.size, v.size))


# ---- math.rs ---------------------------------------------------------------
def quantize_rows_i8(w, rows: int, cols: int):
    w = _f32(w).reshape(rows, cols)
    q = np.empty((rows, cols), np.int8)
    s = np.empty(rows, np.float32)
    lib().orc_quantize_rows_i8(_ptr(w), rows, cols, _ptr(q), _ptr(s))
    return q, s


def matvec_i8(x, q, scales) -> np.ndarray:
    rows, cols = q.shape
    x, scales = _f32(x), _f32(scales)
    q = np.ascontiguousarray(q, np.int8)
    out = np.empty(rows, np.float32)
    lib().orc_matvec_i8(_ptr(out), _ptr(x), _ptr(q), _ptr(scales), rows, cols)
    return out


def matvec_f32(x, w, sequential: bool = False) -> np.ndarray:
    w = _f32(w)
    rows, cols = w.shape
    x = _f32(x)
    out = np.empty(rows, np.float32)
    fn = lib().orc_matvec_f32_sequential if sequential else lib().orc_matvec_f32
    fn(_ptr(out), _ptr(x), _ptr(w), rows, cols)
    return out


def matmat_i8(x_br, q, scales, tile: int = 4) -> np.ndarray:
    """Projection::apply_batched for int8: returns [batch][rows]."""
    rows, cols = q.shape
    x_br = _f32(x_br).reshape(-1, cols)
    batch = x_br.shape[0]
    q = np.ascontiguousarray(q, np.int8)
    scales = _f32(scales)
    stage = np.empty((rows, batch), np.float32)
    lib().orc_matmat_i8(_ptr(stage), _ptr(x_br), _ptr(q), _ptr(scales), batch, rows, cols, tile)
    out = np.empty((batch, rows), np.float32)
    lib().orc_transpose_rb_to_br(_ptr(stage), _ptr(out), rows, batch)
    return out


def matmat_f32(x_br, w, tile: int = 4) -> np.ndarray:
    w = _f32(w)
    rows, cols = w.shape
    x_br = _f32(x_br).reshape(-1, cols)
    batch = x_br.shape[0]
    stage = np.empty((rows, batch), np.float32)
    lib().orc_matmat_f32(_ptr(stage), _ptr(x_br), _ptr(w), batch, rows, cols, tile)
    out = np.empty((batch, rows), np.float32)
    lib().orc_transpose_rb_to_br(_ptr(stage), _ptr(out), rows, batch)
    return out


def bf16_to_f32(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, np.uint16)
    out = np.empty(bits.shape, np.float32)
    lib().orc_pack_bf16_to_f32(_ptr(bits), _ptr(out), bits.size)
    return out


def rms_norm(x, weight, eps: float) -> np.ndarray:
    x = _f32(x).copy()
    weight = _f32(weight)
    lib().orc_rms_norm(_ptr(x), _ptr(weight), x.size, eps)
    return x


def silu(x: float) -> float:
    return lib().orc_silu(x)


def swiglu(x, x_w3) -> np.ndarray:
    x = _f32(x).copy()
    x_w3 = _f32(x_w3)
    lib().orc_swiglu(_ptr(x), _ptr(x_w3), x.size)
    return x


def rope_table(pos: int, head_dim: int, theta: float):
    c = np.empty(head_dim // 2, np.float32)
    s = np.empty(head_dim // 2, np.float32)
    lib().orc_rope_table(pos, head_dim, theta, _ptr(c), _ptr(s))
    return c, s


def rope_rotate(x, cos, sin, style: int = 0) -> np.ndarray:
    x = _f32(x).copy()
    cos, sin = _f32(cos), _f32(sin)
    lib().orc_rope_rotate(_ptr(x), x.size, _ptr(cos), _ptr(sin), style)
    return x


def apply_rope(x, pos: int, theta: float, style: int = 0) -> np.ndarray:
    """math::apply_rope (src/math.rs:375-389) for one head vector."""
    x = _f32(x)
    c, s = rope_table(pos, x.size, theta)
    return rope_rotate(x, c, s, style)


def softmax(x) -> np.ndarray:
    x = _f32(x).copy()
    lib().orc_softmax_in_place(_ptr(x), x.size)
    return x


def argmax(logits) -> int:
    logits = _f32(logits)
    return int(lib().orc_argmax(_ptr(logits), logits.size))


# ---- memory/layout.rs ------------------------------------------------------
def kv_layout(num_layers, num_blocks, block_size, num_kv_heads, head_dim) -> KvLayout:
    return KvLayout(num_layers, num_blocks, block_size, num_kv_heads, head_dim)


def kv_index(layout: KvLayout, layer, block, tok, kv_head, is_value) -> int:
    return lib().orc_kv_index(C.byref(layout), layer, block, tok, kv_head, int(is_value))


def kv_copy_block(layout: KvLayout, cache: np.ndarray, src: int, dst: int) -> None:
    assert cache.dtype == np.float32 and cache.flags.c_contiguous
    if lib().orc_kv_copy_block(C.byref(layout), _ptr(cache), src, dst) != 0:
        raise ValueError("copy_block called with src == dst")


# ---- attention.rs ----------------------------------------------------------
def pack_tables(tables):
    """Lists of physical block ids -> ([B x max_blocks] int32, lens[B])."""
    lens = np.array([len(t) for t in tables], np.int32)
    mb = max(1, int(lens.max()) if len(lens) else 1)
    mat = np.full((len(tables), mb), -1, np.int32)
    for b, t in enumerate(tables):
        mat[b, : len(t)] = t
    return mat, lens


def paged_attention(q, kv_cache, layout: KvLayout, num_heads: int, tables, pos, start, layer: int = 0,
                    heads_per_lane: int | None = None, score_stride: int | None = None) -> np.ndarray:
    """PagedAttention::run (src/attention.rs:141-265): out [B][heads][head_dim]."""
    hd = layout.head_dim
    q = _f32(q).reshape(-1)
    batch = len(tables)
    kv_group = num_heads // layout.num_kv_heads
    mat, lens = pack_tables(tables)
    pos = np.ascontiguousarray(pos, np.int64)
    start = np.ascontiguousarray(start, np.int64)
    widest = int(max([max(0, int(p) + 1 - int(s)) for p, s in zip(pos, start)] + [1]))
    stride = score_stride or widest
    d = heads_per_lane or kv_group
    out = np.full(batch * num_heads * hd, np.nan, np.float32)
    scores = np.full(batch * num_heads * stride, np.nan, np.float32)
    kv_cache = _f32(kv_cache)
    rc = lib().orc_paged_attention_run(
        _ptr(out), _ptr(scores), _ptr(q), _ptr(kv_cache), C.byref(layout), layout.block_size, num_heads, hd,
        kv_group, stride, d, _ptr(mat), mat.shape[1], _ptr(lens), _ptr(pos), _ptr(start), batch, layer)
    if rc != 0:
        raise ValueError("paged attention shape assertion failed")
    return out.reshape(batch, num_heads, hd)


# ---- model.rs --------------------------------------------------------------
class Model:
    """LlamaWeights + the forward entry points, over host arrays.

    ``projections[layer]`` is a dict with keys wq, wk, wv, wo, w1, w2, w3; each
    value is either an f32 ``[rows, cols]`` array (Projection::F32), a uint16
    array of bf16 bits (widened at load like ``pack_bf16_to_f32``), or a tuple
    ``(int8 codes, f32 scales)`` (Projection::Int8).
    """

    ORDER = ("wq", "wk", "wv", "wo", "w1", "w2", "w3")

    def __init__(self, cfg: dict, embed_bf16, final_norm, attention_norm, ffn_norm, projections, lm_head):
        self._keep = []
        self.cfg = ModelConfig(
            cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
            cfg["intermediate_size"], cfg["vocab_size"], cfg["rms_norm_eps"], cfg["rope_theta"],
            -1 if cfg.get("attention_window") is None else cfg["attention_window"], cfg.get("rope_style", 0))
        nl = cfg["num_hidden_layers"]
        self.vocab = cfg["vocab_size"]
        embed = self._hold(np.ascontiguousarray(embed_bf16, np.uint16))
        fnorm = self._hold(_f32(final_norm))
        an = (C.c_void_p * nl)(*[_ptr(self._hold(_f32(a))) for a in attention_norm])
        fn = (C.c_void_p * nl)(*[_ptr(self._hold(_f32(a))) for a in ffn_norm])
        tens = (Tensor * (nl * 7))()
        for l in range(nl):
            for j, k in enumerate(self.ORDER):
                tens[l * 7 + j] = self._tensor(projections[l][k])
        w = ModelWeights(_ptr(embed), _ptr(fnorm), an, fn, tens, self._tensor(lm_head))
        self._keep += [an, fn, tens, w]
        self.handle = lib().orc_model_create(C.byref(self.cfg), C.byref(w))
        self._keep.clear()  # the oracle copies everything at create time

    def _hold(self, a):
        self._keep.append(a)
        return a

    def _tensor(self, t) -> Tensor:
        if isinstance(t, tuple):
            q = self._hold(np.ascontiguousarray(t[0], np.int8))
            s = self._hold(_f32(t[1]))
            return Tensor(INT8, q.shape[0], q.shape[1], _ptr(q), _ptr(s))
        t = np.asarray(t)
        if t.dtype == np.uint16:
            t = self._hold(np.ascontiguousarray(t))
            return Tensor(BF16, t.shape[0], t.shape[1], _ptr(t), None)
        t = self._hold(_f32(t))
        return Tensor(F32, t.shape[0], t.shape[1], _ptr(t), None)

    def __del__(self):
        if getattr(self, "handle", None):
            lib().orc_model_destroy(self.handle)
            self.handle = None

    def weight_bytes(self) -> int:
        return lib().orc_model_weight_bytes(self.handle)

    def forward(self, token: int, pos: int, table, kv_cache: np.ndarray, block_size: int) -> np.ndarray:
        table = np.ascontiguousarray(table, np.int32)
        logits = np.empty(self.vocab, np.float32)
        lib().orc_model_forward(self.handle, token, pos, _ptr(table), table.size, _ptr(kv_cache), kv_cache.size,
                                block_size, _ptr(logits))
        return logits

    def prefill(self, tokens, start_pos: int, table, kv_cache: np.ndarray, block_size: int) -> np.ndarray:
        tokens = np.ascontiguousarray(tokens, np.uint32)
        table = np.ascontiguousarray(table, np.int32)
        logits = np.empty(self.vocab, np.float32)
        rc = lib().orc_model_prefill(self.handle, _ptr(tokens), tokens.size, start_pos, _ptr(table), table.size,
                                     _ptr(kv_cache), kv_cache.size, block_size, _ptr(logits))
        if rc != 0:
            raise ValueError("prefill needs at least one token")
        return logits

    def decode_batch(self, tokens, positions, tables, kv_cache: np.ndarray, block_size: int) -> np.ndarray:
        tokens = np.ascontiguousarray(tokens, np.uint32)
        positions = np.ascontiguousarray(positions, np.int64)
        mat, lens = pack_tables(tables)
        batch = tokens.size
        logits = np.empty((batch, self.vocab), np.float32)
        rc = lib().orc_model_decode_batch(self.handle, _ptr(tokens), _ptr(positions), _ptr(mat), mat.shape[1],
                                          _ptr(lens), batch, _ptr(kv_cache), kv_cache.size, block_size, _ptr(logits))
        if rc != 0:
            raise ValueError("decode_batch_into needs at least one sequence")
        return logits

    def prefill_batched(self, tokens, start_pos: int, table, kv_cache: np.ndarray, block_size: int,
                        chunk_size: int, capacity: int | None = None) -> np.ndarray:
        tokens = np.ascontiguousarray(tokens, np.uint32)
        table = np.ascontiguousarray(table, np.int32)
        logits = np.empty(self.vocab, np.float32)
        rc = lib().orc_model_prefill_batched(self.handle, _ptr(tokens), tokens.size, start_pos, _ptr(table),
                                             table.size, _ptr(kv_cache), kv_cache.size, block_size, chunk_size,
                                             capacity or max(chunk_size, 1), _ptr(logits))
        if rc != 0:
            raise ValueError("prefill needs at least one token")
        return logits
