"""The C-ABI library loads without a GPU and exports exactly what the header
declares; the host-side helpers (layout arithmetic, block tables, loader)
behave like the reference's (src/memory/layout.rs:99-177,
src/memory/block_table.rs:50-61, src/model.rs:65-96)."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "paged_infer_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pi_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def built_lib():
    from paged_infer_b200 import build
    return build.build()


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    names = header_functions()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"


def test_binding_covers_the_header(built_lib):
    from paged_infer_b200 import _lib
    assert sorted(_lib.SIGNATURES) == header_functions()
    _lib.lib()
    assert b"sm_100a" in _lib.lib().pi_version()


def test_no_device_is_a_loud_error_not_a_fallback(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from paged_infer_b200 import api
    with pytest.raises(api.PiError) as e:
        api.Context(0)
    assert "no CPU fallback" in str(e.value) or "CUDA" in str(e.value)


def test_kv_layout_matches_the_oracle_arithmetic(oracle):
    from paged_infer_b200.api import KvLayout
    L = KvLayout(3, 5, 4, 2, 8)
    O = oracle.kv_layout(3, 5, 4, 2, 8)
    assert L.total_floats() == O.total_floats()
    for layer in range(3):
        for blk in (0, 4):
            for tok in (0, 3):
                for h in (0, 1):
                    for v in (False, True):
                        assert L.index(layer, blk, tok, h, v) == oracle.kv_index(O, layer, blk, tok, h, v)


def test_block_table_lookup():
    from paged_infer_b200.api import BlockTable, pack_block_tables
    t = BlockTable([7, 3, 9])
    assert t.get_physical_location(0, 8) == (7, 0)
    assert t.get_physical_location(15, 8) == (3, 7)
    assert t.get_physical_location(23, 8) == (9, 7)
    assert t.get_physical_location(24, 8) is None
    t.remap(1, 11)
    assert t.physical_blocks() == [7, 11, 9] and len(t) == 3
    mat, lens, mb = pack_block_tables([t, BlockTable([2]), BlockTable()])
    assert mb == 3 and lens.tolist() == [3, 1, 0]
    assert mat.tolist() == [[7, 11, 9], [2, -1, -1], [-1, -1, -1]]


def test_loader_reads_the_fixture_and_config(tmp_path):
    from helpers import GOLDEN, load_golden
    from paged_infer_b200.loader import LlamaConfig, bf16_bits_to_f32, f32_to_bf16_bits
    cfg, tokens, golden, hw = load_golden()
    assert (cfg.hidden_size, cfg.head_dim, cfg.kv_dim, cfg.kv_group) == (96, 24, 48, 2)
    assert hw.token_embeddings.shape == (112, 96) and hw.lm_head.shape == (112, 96)
    assert hw.projections[1]["w2"].shape == (96, 192) and hw.projections[0]["wk"].shape == (48, 96)
    w = bf16_bits_to_f32(hw.projections[0]["wq"])
    assert np.array_equal(f32_to_bf16_bits(w), hw.projections[0]["wq"])
    p = tmp_path / "config.json"
    p.write_text('{"hidden_size": 64, "num_attention_heads": 8, "rope_theta": 500000.0}')
    c = LlamaConfig.from_hf_config(str(p))
    assert c.hidden_size == 64 and c.num_key_value_heads == 8 and c.rope_theta == 500000.0 and c.vocab_size == 32000


def test_rust_ffi_is_generated_from_the_header():
    """bindings/rust/src/ffi.rs is a pure function of the header: regenerate and compare, and every function is there."""
    import subprocess
    import sys
    gen = os.path.join(ROOT, "bindings", "rust", "gen_ffi.py")
    assert subprocess.run([sys.executable, gen, "--check"]).returncode == 0, "run python bindings/rust/gen_ffi.py"
    text = open(os.path.join(ROOT, "bindings", "rust", "src", "ffi.rs")).read()
    for n in header_functions():
        assert f"pub fn {n}(" in text, n
