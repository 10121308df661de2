"""Writes tests/golden/golden.npz: small input/output vectors for the hot path, produced by the CPU oracle from seeded inputs.

The reference is Rust and cannot run here, so these are not outputs of the reference itself: the oracle that makes them is
pinned to the reference's own known answers by tests/test_oracle_*.py, and the fixture freezes its results so that a later
change of the oracle or of the CUDA path shows up against a committed file. The known-answer vectors of the reference's
unit tests that the oracle is pinned to are stored alongside (quantiser: rust/crates/quintrit-runtime/src/ops.rs:1968-1992;
row sizes: rust/crates/quintrit-cuda/src/pack.rs:142-149).

Run from the repository root: python tests/golden/make_golden.py
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from quintrit_b200 import synth  # noqa: E402

GEMV_SHAPES = [(33, 161), (64, 320), (96, 3072), (40, 23040)]
MODEL_ARGS = dict(hidden=256, inter=512, layers=2, q_heads=4, kv_heads=2, head_dim=64, vocab=300, ctx=256)
MODEL_TOKENS = 8


def model_spec(arch: int, f32_values: bool) -> dict:
    a = MODEL_ARGS
    return synth.make_model(arch, f32_values, a["hidden"], a["inter"], a["layers"], a["q_heads"], a["kv_heads"], a["head_dim"], a["vocab"], a["ctx"],
                            500000.0, 1e-5, config=41, random_norms=True, tied=(arch == 1))


def main() -> None:
    out = {}
    for i, (rows, cols) in enumerate(GEMV_SHAPES):
        trits = synth.trits(synth.seed_for(40, i, 0, 0), rows * cols)
        act = synth.quantize_int8_np(synth.normal_f32(synth.seed_for(40, i, 0, 2), cols))[0]
        out[f"gemv{i}_planar"] = oracle.pack_planar(trits, rows, cols)
        out[f"gemv{i}_act"] = act
        out[f"gemv{i}_out"] = oracle.gemv_bruteforce(trits, rows, cols, act).astype(np.int32)
    for arch in (0, 1):
        for f32v in (False, True):
            spec = model_spec(arch, f32v)
            ref = oracle.Model(spec)
            toks = synth.prompt_tokens(41, MODEL_TOKENS, spec["vocab"])
            logits = np.stack([ref.forward(int(t), p) for p, t in enumerate(toks)])
            out[f"model_a{arch}_f{int(f32v)}_tokens"] = toks
            out[f"model_a{arch}_f{int(f32v)}_logits_bits"] = logits.view(np.uint32)
    # block-scaled projection
    rng = np.random.default_rng(42)
    rows, cols = 17, 640
    trits = rng.integers(-1, 2, size=(rows, cols)).astype(np.int8)
    wsc = rng.uniform(0.5, 2.0, rows * cols // 64).astype(np.float16).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    qs, d = oracle.quantize_q8_0(x)
    out["bs_trits"], out["bs_wscales"], out["bs_x"], out["bs_codes"], out["bs_scales"] = trits, wsc, x, qs, d
    out["bs_out_bits"] = oracle.gemv_block_scaled(oracle.pack_planar(trits.reshape(-1), rows, cols), wsc, qs, d, rows, cols).view(np.uint32)
    # known answers of the reference's own tests
    out["ref_quant_in"] = np.array([0.5, -1.0, 0.25, 1.0, -0.001], np.float32)
    out["ref_quant_codes"] = np.array([64, -127, 32, 127, 0], np.int8)
    out["ref_quant_scale"] = np.array([127.0], np.float32)
    out["ref_row_bytes_cols"] = np.array([3072, 23040, 160, 161], np.int64)
    out["ref_row_bytes"] = np.array([640, 4608, 32, 64], np.int64)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
