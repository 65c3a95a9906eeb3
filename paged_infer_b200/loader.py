"""Host-side checkpoint reading: the counterpart of ``ModelLoader`` and
``LlamaConfig::from_hf_config`` (reference ``src/model.rs:65-103``, ``:388-455``).

Pure host code (numpy only): it parses a safetensors file holding bf16 tensors
under HuggingFace Llama names and returns raw bf16 bit arrays.  Widening,
quantisation and upload happen in the CUDA library.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field

import numpy as np

ROPE_NEOX = 0
ROPE_INTERLEAVED = 1

QUANT_F32 = "f32"    # reference Quantization::F32 (bf16 checkpoint widened exactly)
QUANT_INT8 = "int8"  # reference Quantization::Int8


@dataclass
class LlamaConfig:
    """Field-for-field ``LlamaConfig`` (reference ``src/model.rs:14-53``)."""

    hidden_size: int = 2048
    num_hidden_layers: int = 22
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    intermediate_size: int = 5632
    vocab_size: int = 32000
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    attention_window: int | None = None
    rope_style: int = ROPE_NEOX
    quantization: str = QUANT_F32

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_hf_config(cls, path: str) -> "LlamaConfig":
        """Read the architecture from a HuggingFace ``config.json``; absent
        fields keep their defaults and ``num_key_value_heads`` falls back to the
        query head count (reference ``src/model.rs:65-96``)."""
        with open(path) as f:
            j = json.load(f)
        d = cls()
        heads = int(j.get("num_attention_heads", d.num_attention_heads))
        return cls(
            hidden_size=int(j.get("hidden_size", d.hidden_size)),
            num_hidden_layers=int(j.get("num_hidden_layers", d.num_hidden_layers)),
            num_attention_heads=heads,
            num_key_value_heads=int(j.get("num_key_value_heads", heads)),
            intermediate_size=int(j.get("intermediate_size", d.intermediate_size)),
            vocab_size=int(j.get("vocab_size", d.vocab_size)),
            rms_norm_eps=float(j.get("rms_norm_eps", d.rms_norm_eps)),
            rope_theta=float(j.get("rope_theta", d.rope_theta)),
        )

    def as_dict(self) -> dict:
        return {k: getattr(self, k) for k in (
            "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
            "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta", "attention_window", "rope_style")}


def read_safetensors(path: str) -> dict:
    """name -> uint16 array of bf16 bits with the stored shape."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        if info["dtype"] != "BF16":
            raise ValueError(f"{name}: only BF16 checkpoints are supported, got {info['dtype']}")
        a, b = info["data_offsets"]
        out[name] = np.frombuffer(raw, dtype="<u2", count=(b - a) // 2, offset=base + a).reshape(info["shape"])
    return out


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """Exact widening (reference ``pack_bf16_to_f32``, ``src/math.rs:66-71``)."""
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bits."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    bias = np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return ((u + bias) >> np.uint32(16)).astype(np.uint16)


@dataclass
class HostWeights:
    """What ``ModelLoader::load_weights`` collects (reference
    ``src/model.rs:398-446``), still as bf16 bits: the CUDA library decides the
    device representation per ``quantization``."""

    token_embeddings: np.ndarray            # [vocab, hidden] bf16 bits
    final_norm: np.ndarray                  # [hidden] f32
    attention_norm: list = field(default_factory=list)   # per layer [hidden] f32
    ffn_norm: list = field(default_factory=list)
    projections: list = field(default_factory=list)      # per layer dict wq..w3 -> bf16 bits [rows, cols]
    lm_head: np.ndarray | None = None       # bf16 bits [vocab, hidden]


def load_weights(path: str, cfg: LlamaConfig) -> HostWeights:
    t = read_safetensors(path)

    def need(name):
        if name not in t:
            raise KeyError(f"missing tensor: {name}")
        return t[name]

    embed = need("model.embed_tokens.weight")
    # Tied embeddings: fall back to the embedding matrix (reference :401-403).
    lm_head = t.get("lm_head.weight", embed)
    hw = HostWeights(token_embeddings=embed, final_norm=bf16_bits_to_f32(need("model.norm.weight")), lm_head=lm_head)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        hw.attention_norm.append(bf16_bits_to_f32(need(f"{p}.input_layernorm.weight")))
        hw.ffn_norm.append(bf16_bits_to_f32(need(f"{p}.post_attention_layernorm.weight")))
        hw.projections.append({
            "wq": need(f"{p}.self_attn.q_proj.weight"),
            "wk": need(f"{p}.self_attn.k_proj.weight"),
            "wv": need(f"{p}.self_attn.v_proj.weight"),
            "wo": need(f"{p}.self_attn.o_proj.weight"),
            "w1": need(f"{p}.mlp.gate_proj.weight"),
            "w2": need(f"{p}.mlp.down_proj.weight"),
            "w3": need(f"{p}.mlp.up_proj.weight"),
        })
    return hw
