"""Shared input generators for the parity tests.

The closed-form generators restate the ones the reference's tests use, so the
same inputs reach the oracle and the CUDA library:
  seq / seq_i8            tests/simd_tests.rs:15-31
  AttnCase                tests/attention_tests.rs:28-84
  load_golden             tests/golden_parity_tests.rs:34-84
"""
from __future__ import annotations

import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def seq(n: int, seed: int) -> np.ndarray:
    i = np.arange(n, dtype=np.uint64)
    t = (i * np.uint64(2654435761) + np.uint64(seed)) & np.uint64(0xFFFFFFFF)
    return ((t % np.uint64(2003)).astype(np.float32) / np.float32(1000.0)) - np.float32(1.0)


def seq_i8(n: int, seed: int) -> np.ndarray:
    i = np.arange(n, dtype=np.uint64)
    t = (i * np.uint64(2246822519) + np.uint64(seed)) & np.uint64(0xFFFFFFFF)
    return ((t % np.uint64(255)).astype(np.int32) - 127).astype(np.int8)


def normal_f32(shape, seed: int, std: float = 1.0) -> np.ndarray:
    return (np.random.default_rng(seed).standard_normal(shape) * std).astype(np.float32)


class AttnCase:
    """One layer of KV, `batch` sequences with `blocks_per_seq` logical blocks of
    which `mapped_blocks` are backed; physical blocks handed out in reverse."""

    def __init__(self, num_heads, num_kv_heads, head_dim, block_size, batch, blocks_per_seq, mapped_blocks,
                 num_layers=1):
        total = blocks_per_seq * batch + 3
        self.num_heads, self.num_kv_heads, self.head_dim, self.block_size = num_heads, num_kv_heads, head_dim, block_size
        self.total_blocks = total
        self.num_layers = num_layers
        handed = list(range(total))[::-1]
        self.tables = [[handed[(b * blocks_per_seq + i) % total] for i in range(mapped_blocks)] for b in range(batch)]
        n = num_layers * total * block_size * num_kv_heads * 2 * head_dim
        self.kv_cache = ((np.arange(n) % 173).astype(np.float32) * np.float32(0.017) - np.float32(1.3)).astype(np.float32)
        nq = batch * num_heads * head_dim
        self.q = ((np.arange(nq) % 91).astype(np.float32) * np.float32(0.031) - np.float32(1.1)).astype(np.float32)

    def starts(self, positions, window):
        return [max(0, p + 1 - window) if window is not None else 0 for p in positions]

    def naive(self, q, tables, positions, starts, layer=0):
        """One head and one token at a time (tests/attention_tests.rs:87-134), in f32."""
        H, KH, D, BS = self.num_heads, self.num_kv_heads, self.head_dim, self.block_size
        g = H // KH
        kv = self.kv_cache.reshape(self.num_layers, self.total_blocks, BS, KH, 2, D)
        q = np.asarray(q, np.float32).reshape(len(tables), H, D)
        out = np.zeros((len(tables), H, D), np.float32)
        scale = np.float32(1.0) / np.sqrt(np.float32(D))
        for b, (tab, pos, st) in enumerate(zip(tables, positions, starts)):
            used = max(0, pos + 1 - st)
            if used == 0:
                continue
            for h in range(H):
                kvh = h // g
                sc = np.full(used, -np.inf, np.float32)
                for si, t in enumerate(range(st, pos + 1)):
                    lb, off = divmod(t, BS)
                    if lb < len(tab):
                        k = kv[layer, tab[lb], off, kvh, 0]
                        acc = np.float32(0)
                        for a, c in zip(q[b, h], k):
                            acc = np.float32(acc + np.float32(a * c))
                        sc[si] = acc * scale
                m = sc.max()
                if not np.isfinite(m):
                    continue
                e = np.exp(sc - m, dtype=np.float32)
                s = np.float32(0)
                for v in e:
                    s = np.float32(s + v)
                w = e * (np.float32(1.0) / max(s, np.float32(1e-12)))
                for si, t in enumerate(range(st, pos + 1)):
                    if w[si] == 0:
                        continue
                    lb, off = divmod(t, BS)
                    if lb < len(tab):
                        out[b, h] += w[si] * kv[layer, tab[lb], off, kvh, 1]
        return out


def load_golden():
    """Config, tokens, golden logits [40,112] and the host weights of the fixture."""
    from paged_infer_b200.loader import LlamaConfig, load_weights

    meta = {}
    with open(os.path.join(GOLDEN, "tiny_llama_meta.txt")) as f:
        for line in f:
            if "=" in line:
                k, v = line.strip().split("=", 1)
                meta[k] = v
    cfg = LlamaConfig(
        hidden_size=int(meta["hidden_size"]), num_hidden_layers=int(meta["num_hidden_layers"]),
        num_attention_heads=int(meta["num_attention_heads"]), num_key_value_heads=int(meta["num_key_value_heads"]),
        intermediate_size=int(meta["intermediate_size"]), vocab_size=int(meta["vocab_size"]),
        rms_norm_eps=float(meta["rms_norm_eps"]), rope_theta=float(meta["rope_theta"]))
    tokens = np.array([int(t) for t in meta["tokens"].split(",")], np.uint32)
    assert tokens.size == int(meta["seq_len"])
    golden = np.fromfile(os.path.join(GOLDEN, "tiny_llama_golden.bin"), "<f4").reshape(tokens.size, cfg.vocab_size)
    hw = load_weights(os.path.join(GOLDEN, "tiny_llama.safetensors"), cfg)
    return cfg, tokens, golden, hw


def compare_logits(actual: np.ndarray, expected: np.ndarray, argmax_fn):
    """(max |delta|, argmax mismatches) as tests/golden_parity_tests.rs:101-120."""
    actual = actual.reshape(expected.shape)
    max_abs = float(np.abs(actual - expected).max())
    mism = sum(int(argmax_fn(a) != argmax_fn(e)) for a, e in zip(actual, expected))
    return max_abs, mism


def oracle_model(oracle, cfg, hw, quant: str = "f32", lm_head_int8: bool = False):
    """Build the oracle model the way the reference loader would (QUANT=f32|int8;
    lm_head stays f32 unless lm_head_int8)."""
    projs = []
    for layer in hw.projections:
        d = {}
        for k, bits in layer.items():
            if quant == "int8":
                w = oracle.bf16_to_f32(bits)
                d[k] = oracle.quantize_rows_i8(w, *w.shape)
            else:
                d[k] = np.ascontiguousarray(bits, np.uint16)
        projs.append(d)
    lm = np.ascontiguousarray(hw.lm_head, np.uint16)
    if lm_head_int8:
        w = oracle.bf16_to_f32(lm)
        lm = oracle.quantize_rows_i8(w, *w.shape)
    return oracle.Model(cfg.as_dict(), hw.token_embeddings, hw.final_norm, hw.attention_norm, hw.ffn_norm, projs, lm)
