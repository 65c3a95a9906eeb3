#!/usr/bin/env python3
"""Regenerate the golden fixtures in this directory from the reference.

Runs only where a checkout of the reference is at hand: pass its directory as the
first argument or in ``PAGED_INFER_REFERENCE``.  It imports the reference's own NumPy generator
``scripts/gen_golden_fixture.py`` (an independent transcription of HuggingFace
``modeling_llama``), calls its ``build_weights`` / ``reference_forward`` with
the seed it uses (20240517) and writes

  tiny_llama.safetensors   bf16 checkpoint in HF tensor layout
  tiny_llama_golden.bin    40 x 112 f32 logits (little endian)
  tiny_llama_meta.txt      config + the 40 token ids
  tiny_llama_interleaved_golden.bin  the same forward under the interleaved
                           rotary convention (the generator computes it to prove
                           the fixture tells the two conventions apart)

and then checks the first three byte-for-byte against the copies the
reference's tests read (``tests/fixtures/``).  The committed files are the
output of this script; tests never need the reference checkout.
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PAGED_INFER_REFERENCE", "")


def main() -> int:
    gen_path = os.path.join(REF, "scripts", "gen_golden_fixture.py")
    if not REF or not os.path.exists(gen_path):
        print(f"reference generator not found at {gen_path}", file=sys.stderr)
        return 1
    sys.dont_write_bytecode = True
    spec = importlib.util.spec_from_file_location("gen_golden_fixture", gen_path)
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)

    rng = np.random.default_rng(20240517)
    tensors = gen.build_weights(rng)
    tokens = rng.integers(0, gen.VOCAB, size=gen.SEQ_LEN, dtype=np.uint32)
    logits = gen.reference_forward(tensors, tokens, interleaved=False)
    inter = gen.reference_forward(tensors, tokens, interleaved=True)

    gen.write_safetensors(os.path.join(HERE, "tiny_llama.safetensors"), tensors)
    with open(os.path.join(HERE, "tiny_llama_golden.bin"), "wb") as f:
        f.write(logits.astype("<f4").tobytes())
    with open(os.path.join(HERE, "tiny_llama_interleaved_golden.bin"), "wb") as f:
        f.write(inter.astype("<f4").tobytes())
    meta = [
        f"hidden_size={gen.HIDDEN}",
        f"num_hidden_layers={gen.LAYERS}",
        f"num_attention_heads={gen.HEADS}",
        f"num_key_value_heads={gen.KV_HEADS}",
        f"intermediate_size={gen.INTERMEDIATE}",
        f"vocab_size={gen.VOCAB}",
        f"rms_norm_eps={gen.EPS}",
        f"rope_theta={gen.THETA}",
        f"seq_len={gen.SEQ_LEN}",
        "tokens=" + ",".join(str(int(t)) for t in tokens),
    ]
    with open(os.path.join(HERE, "tiny_llama_meta.txt"), "w") as f:
        f.write("\n".join(meta) + "\n")

    ok = True
    for name in ("tiny_llama.safetensors", "tiny_llama_golden.bin", "tiny_llama_meta.txt"):
        mine = open(os.path.join(HERE, name), "rb").read()
        theirs = open(os.path.join(REF, "tests", "fixtures", name), "rb").read()
        same = mine == theirs
        ok &= same
        print(f"{name}: {len(mine)} bytes, identical to the reference's fixture: {same}")
    return 0 if ok else 2


if __name__ == "__main__":
    raise SystemExit(main())
