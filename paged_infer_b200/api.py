"""Host-side mirror of the reference's Rust interface for the decode hot path,
over the C ABI of ``libpaged_infer_cuda.so``.

Names, argument meaning and error behaviour follow the reference crate
(``src/model.rs``, ``src/attention.rs``, ``src/memory/layout.rs``,
``src/memory/block_table.rs``, ``src/math.rs``, ``src/sampling.rs``): where
the Rust code asserts, these raise ``PiError`` with ``PI_ERR_INVALID_ARG``.
Host arrays are numpy; the KV pool, the weights and all scratch live in device
memory owned by the library's handles.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import PI_BF16, PI_F32, PI_INT8, PI_SPLIT_COLUMN, PI_SPLIT_NONE, PI_SPLIT_ROW, PiError, check
from .loader import QUANT_F32, QUANT_INT8, HostWeights, LlamaConfig


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def _dev_ptr(t) -> int:
    """Device pointer of a torch CUDA tensor (or a raw int)."""
    return int(t) if isinstance(t, int) else int(t.data_ptr())


class Context:
    """One device, one stream, one host thread (``pi_ctx``).

    ``stream`` is a raw ``cudaStream_t`` (e.g. ``torch.cuda.current_stream().cuda_stream``);
    by default the context creates its own.  With ``tp > 1`` this is rank
    ``rank`` of a tensor-parallel group; ``nccl_id`` is the 128-byte id from
    :func:`nccl_unique_id` on rank 0.
    """

    def __init__(self, device: int = 0, stream: int | None = None, rank: int = 0, tp: int = 1, nccl_id: bytes | None = None):
        L = _lib.lib()
        h = C.c_void_p()
        if tp > 1:
            buf = C.create_string_buffer(nccl_id, 128) if nccl_id is not None else None
            check(L.pi_ctx_create_tp(device, stream, rank, tp, buf, C.byref(h)))
        else:
            check(L.pi_ctx_create(device, stream, C.byref(h)))
        self.handle = h
        self.device, self.rank, self.tp = device, rank, tp

    def close(self):
        if getattr(self, "handle", None) and _lib is not None:   # module globals are gone at interpreter exit
            _lib.lib().pi_ctx_destroy(self.handle)
            self.handle = None

    __del__ = close

    def synchronize(self):
        check(_lib.lib().pi_ctx_synchronize(self.handle), self.handle)

    def kernel_launches(self) -> int:
        return int(_lib.lib().pi_ctx_kernel_launches(self.handle))

    def reset_kernel_launches(self):
        _lib.lib().pi_ctx_reset_kernel_launches(self.handle)

    def profile_begin(self):
        """Start bracketing every launch with CUDA events (per kernel class)."""
        check(_lib.lib().pi_ctx_profile_begin(self.handle), self.handle)

    def profile_end(self) -> dict:
        """{class: (device ms, launches)} since :meth:`profile_begin`."""
        n = len(_lib.PROF_CLASSES)
        ms = (C.c_double * n)()
        cnt = (C.c_uint64 * n)()
        check(_lib.lib().pi_ctx_profile_end(self.handle, ms, cnt), self.handle)
        return {name: (float(ms[i]), int(cnt[i])) for i, name in enumerate(_lib.PROF_CLASSES)}

    def set_option(self, option: int, value: int):
        check(_lib.lib().pi_ctx_set_option(self.handle, option, value), self.handle)

    def tp_peer_export(self, max_floats: int) -> bytes:
        """Allocate this rank's peer-readable exchange buffers (``max_floats`` = max rows x hidden) -> 64-byte handle."""
        buf = C.create_string_buffer(64)
        check(_lib.lib().pi_tp_peer_export(self.handle, max_floats, buf), self.handle)
        return buf.raw

    def tp_peer_import(self, handles) -> None:
        """``handles``: the 64-byte handles of all ranks, in rank order."""
        raw = b"".join(handles)
        if len(raw) != 64 * self.tp:
            raise PiError(_lib.PI_ERR_INVALID_ARG, "one 64-byte handle per rank is needed")
        check(_lib.lib().pi_tp_peer_import(self.handle, C.create_string_buffer(raw, len(raw))), self.handle)

    def tp_peer_base(self) -> int:
        """Device address of this rank's exchange buffers (after :meth:`tp_peer_export`)."""
        return int(_lib.lib().pi_tp_peer_base(self.handle) or 0)

    def tp_peer_import_pointers(self, bases) -> None:
        """Single-process set-up: ``bases`` = :meth:`tp_peer_base` of every rank's context, in rank order."""
        if len(bases) != self.tp:
            raise PiError(_lib.PI_ERR_INVALID_ARG, "one base pointer per rank is needed")
        arr = (C.c_void_p * self.tp)(*[int(b) for b in bases])
        check(_lib.lib().pi_tp_peer_import_pointers(self.handle, arr), self.handle)

    def tp_exchange_add(self, partial_dev, x_dev, rows: int, cols: int) -> None:
        """``x += sum over ranks of partial`` for [rows, cols] device matrices (``pi_tp_exchange_add``)."""
        check(_lib.lib().pi_tp_exchange_add(self.handle, _dev_ptr(partial_dev), _dev_ptr(x_dev), rows, cols), self.handle)


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    check(_lib.lib().pi_nccl_unique_id(buf))
    return buf.raw


def version() -> str:
    return _lib.lib().pi_version().decode()


# ---- math.rs -------------------------------------------------------------------

def quantize_rows_i8(ctx: Context, weight, rows: int, cols: int):
    """``math::quantize_rows_i8`` (src/math.rs:456-469) on the device: (codes [rows, cols] int8, scales [rows] f32)."""
    w = _f32(weight).reshape(rows, cols)
    q = np.empty((rows, cols), np.int8)
    s = np.empty(rows, np.float32)
    check(_lib.lib().pi_quantize_rows_i8(ctx.handle, _ptr(w), rows, cols, _ptr(q), _ptr(s)), ctx.handle)
    return q, s


def rms_norm(ctx: Context, x, weight, eps: float) -> np.ndarray:
    """``math::rms_norm`` (src/math.rs:4-22) per row of ``x``."""
    x = _f32(x).copy()
    weight = _f32(weight)
    rows = 1 if x.ndim == 1 else x.shape[0]
    n = x.shape[-1]
    if weight.size != n:
        raise PiError(_lib.PI_ERR_INVALID_ARG, "Input and weight size mismatch for RMSNorm")
    check(_lib.lib().pi_rms_norm_host(ctx.handle, _ptr(x), _ptr(weight), rows, n, eps), ctx.handle)
    return x


def apply_rope(ctx: Context, x, pos, head_dim: int, rope_theta: float, style: int = 0) -> np.ndarray:
    """``rope_table`` + ``rope_rotate`` (src/math.rs:331-367): ``x`` is [rows, heads*head_dim] (or one vector), ``pos`` per row."""
    x = _f32(x).copy()
    x2 = x.reshape(1, -1) if x.ndim == 1 else x
    pos = _i32(np.atleast_1d(pos))
    heads = x2.shape[1] // head_dim
    check(_lib.lib().pi_rope_host(ctx.handle, _ptr(x2), _ptr(pos), x2.shape[0], heads, head_dim, rope_theta, style), ctx.handle)
    return x


def swiglu(ctx: Context, x, x_w3) -> np.ndarray:
    """``math::swiglu`` (src/math.rs:297-302)."""
    x = _f32(x).copy()
    x_w3 = _f32(x_w3)
    if x.size != x_w3.size:
        raise PiError(_lib.PI_ERR_INVALID_ARG, "SwiGLU input sizes must match")
    check(_lib.lib().pi_swiglu_host(ctx.handle, _ptr(x), _ptr(x_w3), x.size), ctx.handle)
    return x


def argmax(ctx: Context, logits) -> np.ndarray | int:
    """``sampling::argmax`` (src/sampling.rs:140-147): ties go to the last index."""
    l = _f32(logits)
    rows = 1 if l.ndim == 1 else l.shape[0]
    out = np.empty(rows, np.uint32)
    check(_lib.lib().pi_argmax_host(ctx.handle, _ptr(l), rows, l.shape[-1], _ptr(out)), ctx.handle)
    return int(out[0]) if l.ndim == 1 else out


# ---- model.rs: projections ---------------------------------------------------------

class Projection:
    """``Projection::{F32, Int8}`` (src/model.rs:218-291) resident on the device."""

    def __init__(self, ctx: Context, handle):
        self.ctx, self.handle = ctx, handle

    # constructors -------------------------------------------------------------
    @classmethod
    def int8(cls, ctx: Context, codes, scales, split: int = PI_SPLIT_NONE) -> "Projection":
        """``QuantizedLinear {rows, cols, weight, scales}`` from existing codes."""
        q = np.ascontiguousarray(codes, np.int8)
        s = _f32(scales)
        if q.ndim != 2 or s.size != q.shape[0]:
            raise PiError(_lib.PI_ERR_INVALID_ARG, "int8 projection needs [rows, cols] codes and [rows] scales")
        h = C.c_void_p()
        check(_lib.lib().pi_linear_create_i8(ctx.handle, q.shape[0], q.shape[1], _ptr(q), _ptr(s), split, C.byref(h)), ctx.handle)
        return cls(ctx, h)

    @classmethod
    def from_packed(cls, ctx: Context, weight_f32, split: int = PI_SPLIT_NONE) -> "Projection":
        """``QuantizedLinear::from_packed`` (src/model.rs:173-182): quantise on the device."""
        w = _f32(weight_f32)
        h = C.c_void_p()
        check(_lib.lib().pi_linear_create_quantized(ctx.handle, w.shape[0], w.shape[1], _ptr(w), split, C.byref(h)), ctx.handle)
        return cls(ctx, h)

    @classmethod
    def f32(cls, ctx: Context, weight, split: int = PI_SPLIT_NONE) -> "Projection":
        """``PackedLinear`` with f32 weights, or bf16 bits (uint16) kept as bf16."""
        w = np.asarray(weight)
        h = C.c_void_p()
        if w.dtype == np.uint16:
            w = np.ascontiguousarray(w)
            check(_lib.lib().pi_linear_create_bf16(ctx.handle, w.shape[0], w.shape[1], _ptr(w), split, C.byref(h)), ctx.handle)
        else:
            w = _f32(w)
            check(_lib.lib().pi_linear_create_f32(ctx.handle, w.shape[0], w.shape[1], _ptr(w), split, C.byref(h)), ctx.handle)
        return cls(ctx, h)

    @classmethod
    def from_tensor(cls, ctx: Context, bf16_bits, quantization: str) -> "Projection":
        """``Projection::from_tensor`` (src/model.rs:225-231) for a bf16 checkpoint tensor."""
        if quantization == QUANT_INT8:
            from .loader import bf16_bits_to_f32
            return cls.from_packed(ctx, bf16_bits_to_f32(np.asarray(bf16_bits)))
        return cls.f32(ctx, np.asarray(bf16_bits, np.uint16))

    def close(self):
        if getattr(self, "handle", None) and _lib is not None:   # module globals are gone at interpreter exit
            _lib.lib().pi_linear_destroy(self.handle)
            self.handle = None

    __del__ = close

    # accessors ----------------------------------------------------------------
    def rows(self) -> int:
        return int(_lib.lib().pi_linear_rows(self.handle))

    def cols(self) -> int:
        return int(_lib.lib().pi_linear_cols(self.handle))

    def weight_bytes(self) -> int:
        return int(_lib.lib().pi_linear_weight_bytes(self.handle))

    def is_int8(self) -> bool:
        return _lib.lib().pi_linear_kind(self.handle) == PI_INT8

    def read_i8(self):
        """This device's int8 codes and scales."""
        rows, cols = self.rows(), self.cols()
        q = np.empty((rows, cols), np.int8)
        s = np.empty(rows, np.float32)
        check(_lib.lib().pi_linear_read_i8(self.ctx.handle, self.handle, _ptr(q), _ptr(s)), self.ctx.handle)
        return q, s

    # application ----------------------------------------------------------------
    def apply_parallel(self, x) -> np.ndarray:
        """``Projection::apply_parallel``: one activation vector -> [rows]."""
        x = _f32(x)
        if x.size != self.cols():
            raise PiError(_lib.PI_ERR_INVALID_ARG, f"input has {x.size} elements, projection has {self.cols()} columns")
        out = np.empty(self.rows(), np.float32)
        check(_lib.lib().pi_linear_apply_host(self.ctx.handle, self.handle, _ptr(x), _ptr(out), 1), self.ctx.handle)
        return out

    def apply_batched(self, x_br, batch: int | None = None) -> np.ndarray:
        """``Projection::apply_batched`` (src/model.rs:247-259): [batch, cols] -> [batch, rows]."""
        x = _f32(x_br).reshape(-1, self.cols())
        batch = x.shape[0] if batch is None else batch
        if batch < 1 or x.shape[0] != batch:
            raise PiError(_lib.PI_ERR_INVALID_ARG, "x_br must hold batch * cols elements and batch >= 1")
        out = np.empty((batch, self.rows()), np.float32)
        check(_lib.lib().pi_linear_apply_host(self.ctx.handle, self.handle, _ptr(x), _ptr(out), batch), self.ctx.handle)
        return out

    def apply_device(self, x_dev, out_dev, batch: int) -> None:
        """Device-resident ``apply_batched``: ``x_dev`` [batch, cols], ``out_dev`` [batch, rows] (torch CUDA tensors or raw pointers)."""
        check(_lib.lib().pi_linear_apply(self.ctx.handle, self.handle, _dev_ptr(x_dev), _dev_ptr(out_dev), batch), self.ctx.handle)


    def apply_device_noalloc(self, x_dev, out_dev, batch: int) -> None:
        """``apply_device`` through the entry point that allocates nothing (``pi_linear_apply_noalloc``).

        For callers that cannot let the library grow its scratch while they run a projection: code inside a
        CUDA stream capture, latency-bound loops, embedders that own all device memory.  It works out of a
        fixed scratch area that is part of the library, so it only takes int8 projections with a multiple of
        128 columns (at most 8192) and 1..64 activation rows; anything larger raises ``PiError``.  Calls that
        overlap on the GPU share that area and must be ordered by the caller.
        """
        check(_lib.lib().pi_linear_apply_noalloc(self.ctx.handle, self.handle, _dev_ptr(x_dev), _dev_ptr(out_dev), batch), self.ctx.handle)


QuantizedLinear = Projection
PackedLinear = Projection


# ---- memory/layout.rs, memory/block_table.rs ---------------------------------------------

class KvLayout:
    """``KvLayout`` (src/memory/layout.rs:18-97): the address arithmetic of the reference's flat cache."""

    def __init__(self, num_layers: int, num_blocks: int, block_size: int, num_kv_heads: int, head_dim: int):
        self.num_layers, self.num_blocks, self.block_size = num_layers, num_blocks, block_size
        self.num_kv_heads, self.head_dim = num_kv_heads, head_dim

    def total_floats(self) -> int:
        return self.num_layers * self.num_blocks * self.block_stride()

    def block_stride(self) -> int:
        return self.block_size * self.num_kv_heads * 2 * self.head_dim

    def index(self, layer: int, phys_block: int, token_offset: int, kv_head: int, is_value: bool) -> int:
        return ((((layer * self.num_blocks + phys_block) * self.block_size + token_offset) * self.num_kv_heads + kv_head) * 2
                + int(is_value)) * self.head_dim

    def as_c(self) -> _lib.KvLayoutC:
        return _lib.KvLayoutC(self.num_layers, self.num_blocks, self.block_size, self.num_kv_heads, self.head_dim)


class BlockTable:
    """``BlockTable`` (src/memory/block_table.rs:28-93): logical -> physical block ids."""

    def __init__(self, blocks=()):
        self.logical_to_physical = [int(b) for b in blocks]

    def append_block(self, physical_block: int):
        self.logical_to_physical.append(int(physical_block))

    def get_physical_location(self, logical_token_idx: int, block_size: int):
        lb, off = divmod(logical_token_idx, block_size)
        if lb >= len(self.logical_to_physical):
            return None
        return self.logical_to_physical[lb], off

    def remap(self, logical_block_idx: int, block: int):
        self.logical_to_physical[logical_block_idx] = int(block)

    def physical_blocks(self):
        return list(self.logical_to_physical)

    def __len__(self):
        return len(self.logical_to_physical)


class PackedBlockTables:
    """Block tables of a batch kept as the arrays the library takes: ``mat`` int32 [B, width] (physical ids, -1 =
    unmapped) and ``lens`` int32 [B].  An engine that appends / remaps single entries as its sequences grow updates
    these in place instead of flattening Python lists on every step."""

    def __init__(self, batch: int, width: int):
        self.mat = np.full((batch, max(width, 1)), -1, np.int32)
        self.lens = np.zeros(batch, np.int32)

    def __len__(self):
        return self.mat.shape[0]

    def set_row(self, b: int, blocks):
        n = len(blocks)
        self._grow(n)
        self.mat[b, :n] = blocks
        self.mat[b, n:] = -1
        self.lens[b] = n

    def append(self, b: int, block: int):
        n = int(self.lens[b])
        self._grow(n + 1)
        self.mat[b, n] = block
        self.lens[b] = n + 1

    def remap(self, b: int, logical: int, block: int):
        self.mat[b, logical] = block

    def _grow(self, width: int):
        if width > self.mat.shape[1]:
            wider = np.full((self.mat.shape[0], max(width, 2 * self.mat.shape[1])), -1, np.int32)
            wider[:, :self.mat.shape[1]] = self.mat
            self.mat = wider


def pack_block_tables(tables):
    """[BlockTable | sequence of ids] or PackedBlockTables -> (int32 [B, max_blocks], int32 lens [B], max_blocks)."""
    if isinstance(tables, PackedBlockTables):
        mb = int(tables.lens.max()) if len(tables) else 0
        return np.ascontiguousarray(tables.mat[:, :max(mb, 1)]), tables.lens, mb
    rows = [t.logical_to_physical if isinstance(t, BlockTable) else list(t) for t in tables]
    lens = np.array([len(r) for r in rows], np.int32)
    mb = int(lens.max()) if len(rows) and lens.max() > 0 else 0
    mat = np.full((len(rows), max(mb, 1)), -1, np.int32)
    for b, r in enumerate(rows):
        mat[b, :len(r)] = r
    return mat, lens, mb


class KvCache:
    """The engine's ``kv_cache`` (src/engine.rs:206-207) as a device-resident pool."""

    def __init__(self, ctx: Context, layout: KvLayout):
        self.ctx, self.layout = ctx, layout
        h = C.c_void_p()
        c = layout.as_c()
        check(_lib.lib().pi_kv_pool_create(ctx.handle, C.byref(c), C.byref(h)), ctx.handle)
        self.handle = h

    def close(self):
        if getattr(self, "handle", None) and _lib is not None:   # module globals are gone at interpreter exit
            _lib.lib().pi_kv_pool_destroy(self.handle)
            self.handle = None

    __del__ = close

    def bytes(self) -> int:
        return int(_lib.lib().pi_kv_pool_bytes(self.handle))

    def copy_block(self, src: int, dst: int):
        """``KvLayout::copy_block`` (src/memory/layout.rs:82-96)."""
        check(_lib.lib().pi_kv_copy_block(self.ctx.handle, self.handle, src, dst), self.ctx.handle)

    def upload(self, cache):
        """Fill the pool from a host array in the reference's layout."""
        c = _f32(cache).reshape(-1)
        if c.size != self.layout.total_floats():
            raise PiError(_lib.PI_ERR_INVALID_ARG, "cache length does not match the layout")
        check(_lib.lib().pi_kv_upload(self.ctx.handle, self.handle, _ptr(c)), self.ctx.handle)

    def download(self) -> np.ndarray:
        """The pool as a host array in the reference's layout."""
        out = np.empty(self.layout.total_floats(), np.float32)
        check(_lib.lib().pi_kv_download(self.ctx.handle, self.handle, _ptr(out)), self.ctx.handle)
        return out

    def fill_normal(self, seed: int, std: float = 1.0):
        """Synthetic N(0, std) contents for benchmarks."""
        check(_lib.lib().pi_kv_fill_normal(self.ctx.handle, self.handle, seed, std), self.ctx.handle)

    def write_token(self, layer: int, block: int, tok: int, k, v):
        k, v = _f32(k), _f32(v)
        check(_lib.lib().pi_kv_write_token(self.ctx.handle, self.handle, layer, block, tok, _ptr(k), _ptr(v)), self.ctx.handle)

    def read_token(self, layer: int, block: int, tok: int):
        n = self.layout.num_kv_heads * self.layout.head_dim
        k, v = np.empty(n, np.float32), np.empty(n, np.float32)
        check(_lib.lib().pi_kv_read_token(self.ctx.handle, self.handle, layer, block, tok, _ptr(k), _ptr(v)), self.ctx.handle)
        return k, v


# ---- attention.rs -----------------------------------------------------------------------------

class AttnEntry:
    """``AttnEntry`` (src/attention.rs:58-85): attends ``start..=pos`` of ``block_table``."""

    def __init__(self, block_table, pos: int, window: int | None = None, start: int | None = None):
        self.block_table = block_table
        self.pos = pos
        self.start = start if start is not None else max(0, pos + 1 - window) if window is not None else 0

    def window_len(self) -> int:
        return max(0, self.pos + 1 - self.start)


class PagedAttention:
    """``PagedAttention`` (src/attention.rs:89-265).  ``score_stride`` and
    ``heads_per_lane`` are CPU scheduling parameters with no device meaning and
    are accepted and ignored."""

    def __init__(self, layout: KvLayout, num_heads: int, score_stride: int | None = None, heads_per_lane: int | None = None):
        self.layout, self.num_heads = layout, num_heads

    def run_device(self, q_dev, out_dev, kv_cache: KvCache, entries, layer: int = 0) -> None:
        """Same as ``run`` with q / out resident on the device (objects with ``data_ptr()``, dense f32
        [entries][num_heads][head_dim]); asynchronous on the context's stream."""
        B = len(entries)
        if B == 0:
            return
        stride = self.num_heads * self.layout.head_dim
        mat, lens, mb = pack_block_tables([e.block_table for e in entries])
        pos = _i32([e.pos for e in entries])
        start = _i32([e.start for e in entries])
        check(_lib.lib().pi_paged_attention(kv_cache.ctx.handle, kv_cache.handle, layer, self.num_heads,
                                            _dev_ptr(q_dev), stride, _dev_ptr(out_dev), stride,
                                            _ptr(mat), mb if mb else 0, _ptr(lens), _ptr(pos), _ptr(start), B),
              kv_cache.ctx.handle)

    def run(self, q, kv_cache: KvCache, entries, layer: int = 0) -> np.ndarray:
        """out [entries, num_heads, head_dim] for q of the same shape."""
        hd = self.layout.head_dim
        B = len(entries)
        q = _f32(q).reshape(-1)
        if q.size != B * self.num_heads * hd:
            raise PiError(_lib.PI_ERR_INVALID_ARG, "q must be [entries][num_heads][head_dim]")
        out = np.zeros((B, self.num_heads, hd), np.float32)
        if B == 0:
            return out
        mat, lens, mb = pack_block_tables([e.block_table for e in entries])
        pos = _i32([e.pos for e in entries])
        start = _i32([e.start for e in entries])
        check(_lib.lib().pi_paged_attention_host(kv_cache.ctx.handle, kv_cache.handle, layer, self.num_heads, _ptr(q), _ptr(out),
                                                 _ptr(mat), mb if mb else 0, _ptr(lens), _ptr(pos), _ptr(start), B),
              kv_cache.ctx.handle)
        return out


# ---- model.rs: forward ---------------------------------------------------------------------------

class LlamaWeights:
    """``LlamaWeights`` + its forward entry points (src/model.rs:380-386, :585-1255) on the device.

    ``quantization`` follows the reference loader: ``"int8"`` quantises the seven
    projections of every layer and leaves the LM head in its checkpoint
    precision unless ``lm_head_int8`` is set.  ``projections`` may also be given
    directly as per-layer dicts of ``(codes, scales)`` tuples / f32 arrays /
    bf16-bit arrays.
    """

    ORDER = ("wq", "wk", "wv", "wo", "w1", "w2", "w3")

    def __init__(self, ctx: Context, config: LlamaConfig, weights: HostWeights, max_batch: int = 32,
                 max_positions: int = 4096, lm_head_int8: bool = False, lm_head=None):
        self.ctx, self.config = ctx, config
        keep = []

        def tensor(t, quantize: bool) -> _lib.TensorC:
            if isinstance(t, tuple):
                q = np.ascontiguousarray(t[0], np.int8)
                s = _f32(t[1])
                keep.extend((q, s))
                return _lib.TensorC(PI_INT8, 0, q.shape[0], q.shape[1], _ptr(q), _ptr(s))
            a = np.asarray(t)
            if a.dtype == np.uint16:
                a = np.ascontiguousarray(a)
                keep.append(a)
                return _lib.TensorC(PI_BF16, int(quantize), a.shape[0], a.shape[1], _ptr(a), None)
            a = _f32(a)
            keep.append(a)
            return _lib.TensorC(PI_F32, int(quantize), a.shape[0], a.shape[1], _ptr(a), None)

        nl = config.num_hidden_layers
        quant = config.quantization == QUANT_INT8
        cfg = _lib.ModelConfigC(config.hidden_size, nl, config.num_attention_heads, config.num_key_value_heads,
                                config.intermediate_size, config.vocab_size, config.rms_norm_eps, config.rope_theta,
                                -1 if config.attention_window is None else config.attention_window, config.rope_style,
                                max_batch, max_positions)
        embed = np.ascontiguousarray(weights.token_embeddings, np.uint16)
        fnorm = _f32(weights.final_norm)
        an = [_f32(a) for a in weights.attention_norm]
        fn = [_f32(a) for a in weights.ffn_norm]
        keep.extend([embed, fnorm] + an + fn)
        an_p = (C.c_void_p * nl)(*[_ptr(a) for a in an])
        fn_p = (C.c_void_p * nl)(*[_ptr(a) for a in fn])
        tens = (_lib.TensorC * (nl * 7))()
        for l in range(nl):
            for j, k in enumerate(self.ORDER):
                tens[l * 7 + j] = tensor(weights.projections[l][k], quant)
        head = lm_head if lm_head is not None else weights.lm_head
        w = _lib.ModelWeightsC(_ptr(embed), _ptr(fnorm), an_p, fn_p, tens, tensor(head, lm_head_int8))
        h = C.c_void_p()
        check(_lib.lib().pi_model_create(ctx.handle, C.byref(cfg), C.byref(w), C.byref(h)), ctx.handle)
        self.handle = h
        self.max_batch = max_batch

    @classmethod
    def synthetic(cls, ctx: Context, config: LlamaConfig, seed: int, std: float = 0.02, quant: int = PI_INT8,
                  lm_head_kind: int = PI_INT8, max_batch: int = 32, max_positions: int = 4096) -> "LlamaWeights":
        """Random-init N(0, std) weights generated and quantised on the device."""
        self = cls.__new__(cls)
        self.ctx, self.config, self.max_batch = ctx, config, max_batch
        cfg = _lib.ModelConfigC(config.hidden_size, config.num_hidden_layers, config.num_attention_heads,
                                config.num_key_value_heads, config.intermediate_size, config.vocab_size,
                                config.rms_norm_eps, config.rope_theta,
                                -1 if config.attention_window is None else config.attention_window, config.rope_style,
                                max_batch, max_positions)
        h = C.c_void_p()
        check(_lib.lib().pi_model_create_synthetic(ctx.handle, C.byref(cfg), seed, std, quant, lm_head_kind, C.byref(h)), ctx.handle)
        self.handle = h
        return self

    def close(self):
        if getattr(self, "handle", None) and _lib is not None:   # module globals are gone at interpreter exit
            _lib.lib().pi_model_destroy(self.handle)
            self.handle = None

    __del__ = close

    def weight_bytes(self) -> int:
        return int(_lib.lib().pi_model_weight_bytes(self.handle))

    def kv_layout(self, num_blocks: int, block_size: int) -> KvLayout:
        """``LlamaConfig::kv_layout`` (src/model.rs:122-130), per tensor-parallel rank."""
        c = self.config
        return KvLayout(c.num_hidden_layers, num_blocks, block_size, c.num_key_value_heads // self.ctx.tp, c.head_dim)

    def decode_batch_into(self, tokens, positions, block_tables, kv_cache: KvCache, want_logits: bool = True,
                          want_argmax: bool = False):
        """``decode_batch_into`` (src/model.rs:1184-1207).  Returns logits [B, vocab], greedy ids [B], or both."""
        tokens = np.ascontiguousarray(tokens, np.uint32)
        positions = _i32(positions)
        B = tokens.size
        if positions.size != B or len(block_tables) != B:
            raise PiError(_lib.PI_ERR_INVALID_ARG, "tokens, positions and block_tables must have one entry per sequence")
        mat, lens, mb = pack_block_tables(block_tables)
        logits = np.empty((B, self.config.vocab_size), np.float32) if want_logits else None
        ids = np.empty(B, np.uint32) if want_argmax else None
        check(_lib.lib().pi_model_decode_batch(self.ctx.handle, self.handle, kv_cache.handle, _ptr(tokens), _ptr(positions),
                                               _ptr(mat), mb, _ptr(lens), B,
                                               _ptr(logits) if want_logits else None, _ptr(ids) if want_argmax else None),
              self.ctx.handle)
        if want_logits and want_argmax:
            return logits, ids
        return logits if want_logits else ids

    def decode_batch_rows(self, tokens, positions, block_tables, kv_cache: KvCache, logit_rows):
        """One batched step that returns the greedy ids of all rows and the full logits of ``logit_rows`` only
        (what Engine::run_groups reads per sequence, src/engine.rs:742-755): ``(logits [len(logit_rows), vocab], ids [B])``."""
        tokens = np.ascontiguousarray(tokens, np.uint32)
        positions = _i32(positions)
        B = tokens.size
        mat, lens, mb = pack_block_tables(block_tables)
        rows = _i32(list(logit_rows))
        logits = np.empty((rows.size, self.config.vocab_size), np.float32)
        ids = np.empty(B, np.uint32)
        check(_lib.lib().pi_model_decode_batch_rows(self.ctx.handle, self.handle, kv_cache.handle, _ptr(tokens), _ptr(positions),
                                                    _ptr(mat), mb, _ptr(lens), B, _ptr(rows) if rows.size else None, int(rows.size),
                                                    _ptr(logits) if rows.size else None, _ptr(ids)), self.ctx.handle)
        return logits, ids

    def decode_multi(self, tokens, positions, block_tables, kv_cache: KvCache, n_steps: int) -> np.ndarray:
        """``n_steps`` greedy decode steps without host round trips; returns token ids [n_steps, B]."""
        tokens = np.ascontiguousarray(tokens, np.uint32)
        positions = _i32(positions)
        B = tokens.size
        mat, lens, mb = pack_block_tables(block_tables)
        out = np.empty((n_steps, B), np.uint32)
        check(_lib.lib().pi_model_decode_multi(self.ctx.handle, self.handle, kv_cache.handle, _ptr(tokens), _ptr(positions),
                                               _ptr(mat), mb, _ptr(lens), B, n_steps, _ptr(out)), self.ctx.handle)
        return out

    def forward(self, token_id: int, pos: int, block_table, kv_cache: KvCache) -> np.ndarray:
        """``LlamaWeights::forward`` (src/model.rs:630-652): one token, logits [vocab]."""
        return self.decode_batch_into([token_id], [pos], [block_table], kv_cache)[0]

    def prefill_batched(self, tokens, start_pos: int, block_table, kv_cache: KvCache, chunk_size: int,
                        want_argmax: bool = False):
        """``prefill_batched`` (src/model.rs:1222-1255): logits [vocab] of the last prompt position."""
        tokens = np.ascontiguousarray(tokens, np.uint32)
        table = _i32(block_table.logical_to_physical if isinstance(block_table, BlockTable) else list(block_table))
        logits = np.empty(self.config.vocab_size, np.float32)
        ids = np.empty(1, np.uint32)
        check(_lib.lib().pi_model_prefill(self.ctx.handle, self.handle, kv_cache.handle, _ptr(tokens), tokens.size, start_pos,
                                          _ptr(table) if table.size else None, table.size, chunk_size, _ptr(logits),
                                          _ptr(ids) if want_argmax else None), self.ctx.handle)
        return (logits, int(ids[0])) if want_argmax else logits

    def prefill(self, tokens, start_pos: int, block_table, kv_cache: KvCache) -> np.ndarray:
        """``LlamaWeights::prefill`` (src/model.rs:700-722): token by token."""
        return self.prefill_batched(tokens, start_pos, block_table, kv_cache, 1)
