"""ctypes binding of ``libpaged_infer_host.so``: the engine's host-side block bookkeeping
(``include/paged_infer_memory.hpp``, a C++ restatement of the reference's ``src/memory/*.rs``) behind a C ABI.

``KvCacheManager`` mirrors the reference type of that name (src/memory/kv_cache_manager.rs:116-345): admission with
prefix reuse through the chained block hash, publishing, forking, copy-on-write before a write into a shared
block.  ``prepare_step`` is what ``Engine::plan_step`` does for a batch (src/engine.rs:612-699) and returns the
block tables in the packed form the device library takes.  Host code only: no GPU is needed to use it.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpaged_infer_host.so")

_P, _SZ, _I, _U64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint64
SIGNATURES = {
    "pih_create": (_P, [_SZ, _SZ, _I]),
    "pih_destroy": (None, [_P]),
    "pih_admit": (C.c_long, [_P, _SZ, _P, _SZ, _U64]),
    "pih_publish": (C.c_long, [_P, _SZ]),
    "pih_fork": (_I, [_P, _SZ, _SZ, _U64]),
    "pih_release": (None, [_P, _SZ]),
    "pih_table": (C.c_long, [_P, _SZ, _P, _SZ]),
    "pih_prepare_step": (C.c_long, [_P, _P, _P, _I, _U64, _P, _I, _P, _P]),
    "pih_stats": (None, [_P, _P]),
}
_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m paged_infer_b200.build`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class OutOfBlocks(RuntimeError):
    pass


class KvCacheManager:
    def __init__(self, num_blocks: int, block_size: int, prefix_cache: bool = True):
        self.handle = lib().pih_create(num_blocks, block_size, int(prefix_cache))
        if not self.handle:
            raise ValueError("num_blocks and block_size must be positive")
        self.block_size = block_size

    def close(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.pih_destroy(self.handle)
            self.handle = None

    __del__ = close

    def admit(self, seq_id: int, tokens, tick: int = 0) -> int:
        """-> number of leading prompt tokens found in the prefix cache (prefill resumes there)."""
        t = np.ascontiguousarray(tokens, np.uint32)
        n = lib().pih_admit(self.handle, seq_id, t.ctypes.data, t.size, tick)
        if n < 0:
            raise OutOfBlocks(f"the pool cannot house a prompt of {t.size} tokens")
        return int(n)

    def publish_prompt_blocks(self, seq_id: int) -> int:
        return int(lib().pih_publish(self.handle, seq_id))

    def fork(self, parent_seq: int, child_seq: int, tick: int = 0) -> None:
        if lib().pih_fork(self.handle, parent_seq, child_seq, tick) != 0:
            raise KeyError(f"cannot fork sequence {parent_seq} into {child_seq}")

    def release_sequence(self, seq_id: int) -> None:
        lib().pih_release(self.handle, seq_id)

    def table(self, seq_id: int) -> list:
        n = lib().pih_table(self.handle, seq_id, None, 0)
        if n < 0:
            raise KeyError(seq_id)
        out = np.empty(max(n, 1), np.int32)
        lib().pih_table(self.handle, seq_id, out.ctypes.data, n)
        return out[:n].tolist()

    def prepare_step(self, seq_ids: np.ndarray, positions: np.ndarray, tables: np.ndarray, lens: np.ndarray, cow: np.ndarray,
                     tick: int = 0) -> int:
        """Settle memory for one batched forward; fills ``tables`` [B, width] / ``lens`` [B] in place and returns the
        number of copy-on-write copies, whose (src, dst) pairs are the first entries of ``cow`` ([B, 2] int32)."""
        B, width = tables.shape
        n = lib().pih_prepare_step(self.handle, seq_ids.ctypes.data, positions.ctypes.data, B, tick, tables.ctypes.data, width,
                                   lens.ctypes.data, cow.ctypes.data)
        if n == -1:
            raise OutOfBlocks("no block left for the step")
        if n < 0:
            raise ValueError("a block table is wider than the packed matrix" if n == -2 else "unknown sequence id")
        return int(n)

    def stats(self) -> dict:
        out = (C.c_uint64 * 8)()
        lib().pih_stats(self.handle, out)
        keys = ("prefix_hits", "prefix_misses", "prefix_tokens_saved", "_", "cow_copies", "free_blocks", "total_blocks", "live_sequences")
        return {k: int(v) for k, v in zip(keys, out) if k != "_"}
