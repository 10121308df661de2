"""Generates fixtures with the reference's OWN GGUF writer (run where the reference tree is available; needs no GPU).

    python tests/golden/make_golden_ref_builder.py /path/to/reference

The reference's Python tests build their models with rust/crates/quintrit-py/tests/gguf_builder.py (write_gguf, pack_i2_s,
pack_tq2_0, tiny_vocab, write_tiny_model). This script imports that module from the reference tree, unmodified, and keeps
what it writes:

  ref_tiny_model.gguf       write_tiny_model(seed 7): the two-layer llama-style model (hidden 128, 4 heads of 32, 2 KV heads,
                            FFN 256, 261 byte-level BPE tokens with three merges, BOS / EOS, context 64, I2_S projections
                            with scale 0.05) that the reference's runtime tests, its C test and its GPU parity test load
  ref_builder_payloads.npz  a seeded trit matrix of 96 x 256 as pack_i2_s packs it (scale 0.125) and one of 4 x 256 as
                            pack_tq2_0 packs it (scale 0.5) - the shapes and scales of the reference's format test
                            (quintrit-py/tests/test_format.py) - with the trits themselves, and the tiny vocabulary

The files pin this repository's readers and decoders (oracle and library) to bytes the reference's code wrote. The
reference's runtime itself (Rust) cannot be built in this environment, so what the model should generate comes from the
CPU oracle; the byte-level facts (tensor payloads, directory, vocabulary, merges) come from the reference.
"""
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def main() -> None:
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QUINTRIT_REFERENCE", ""))
    builder_dir = ref / "rust" / "crates" / "quintrit-py" / "tests"
    if not (builder_dir / "gguf_builder.py").exists():
        raise SystemExit(f"no gguf_builder.py under {builder_dir}")
    sys.path.insert(0, str(builder_dir))
    import gguf_builder as gb  # the reference's module, imported where it lies

    gb.write_tiny_model(HERE / "ref_tiny_model.gguf", seed=7)
    rng = np.random.default_rng(20240611)
    i2s = rng.integers(-1, 2, size=(96, 256)).astype(np.int8)
    tq2 = rng.integers(-1, 2, size=(4, 256)).astype(np.int8)
    tokens, merges, bos, eos = gb.tiny_vocab()
    np.savez_compressed(
        HERE / "ref_builder_payloads.npz",
        i2s_trits=i2s, i2s_payload=np.frombuffer(gb.pack_i2_s(i2s, 0.125), np.uint8),
        tq2_trits=tq2, tq2_payload=np.frombuffer(gb.pack_tq2_0(tq2, 0.5), np.uint8),
        vocab=np.array([t.encode("utf-8") for t in tokens], dtype=object).astype("S8"),
        merges=np.array([m.encode("utf-8") for m in merges], dtype=object).astype("S12"), bos=bos, eos=eos,
        dims=np.array([gb.HIDDEN, gb.FFN, gb.HEADS, gb.KV_HEADS, gb.LAYERS, gb.CONTEXT]),
    )
    print("wrote", HERE / "ref_tiny_model.gguf", (HERE / "ref_tiny_model.gguf").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
