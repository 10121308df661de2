"""The oracle's vector forms (oracle/qt_oracle_fast.c: eight lanes of the reference's AVX2 order per register) against its
portable loops, bit for bit: half and bfloat dot products (rust/crates/quintrit-runtime/src/ops.rs:970-1014, 565-595,
688-712), both attention accumulations (attention.rs:402-469), the block-scaled row product
(rust/crates/quintrit-core/src/block_scaled.rs:175-202) with every byte value, and whole-token logits."""
import ctypes as C

import numpy as np
import pytest

from quintrit_b200 import synth


def _both(oracle, fn):
    l = oracle.mlib()
    l.qto_fast_enable(0)
    a = fn()
    l.qto_fast_enable(1)
    fast = bool(l.qto_fast_available())
    b = fn()
    return a, b, fast


def _bits(x):
    return np.asarray(x, np.float32).reshape(-1).view(np.uint32)


@pytest.mark.parametrize("n", [32, 64, 100, 256, 3072, 3079])
def test_dot_products(oracle, n):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 3).astype(np.float16).view(np.uint16)
    y = (rng.standard_normal(n) * 3).astype(np.float16).view(np.uint16)
    yf = (rng.standard_normal(n) * 3).astype(np.float32)
    xb = oracle.f32_to_bf16_bits(rng.standard_normal(n).astype(np.float32))
    yb = oracle.f32_to_bf16_bits(rng.standard_normal(n).astype(np.float32))
    for fn in (lambda: oracle.vec_dot_f16(x, y), lambda: oracle.vec_dot_f16_f32(x, yf), lambda: oracle.vec_dot_bf16(xb, yb)):
        a, b, _ = _both(oracle, fn)
        assert _bits(a)[0] == _bits(b)[0]


@pytest.mark.parametrize("f32_values", [False, True])
@pytest.mark.parametrize("hd,seq", [(64, 37), (128, 300), (256, 700), (96, 1100)])
def test_attention(oracle, f32_values, hd, seq):
    rng = np.random.default_rng(hd + seq)
    ctx = (seq + 255) // 256 * 256
    k = (rng.standard_normal((ctx, hd)) * 2).astype(np.float16).view(np.uint16)
    v = (rng.standard_normal((ctx, hd)) * 2).astype(np.float16).view(np.uint16)
    q = rng.standard_normal(hd).astype(np.float32)
    a, b, _ = _both(oracle, lambda: oracle.attend_head(q, k, v, hd, seq, ctx, hd, 1.0 / np.sqrt(hd), f32_values))
    assert np.array_equal(_bits(a), _bits(b))


@pytest.mark.parametrize("cols", [64, 160 * 2, 640, 3072, 23040])
def test_block_scaled_rows_with_every_byte_value(oracle, cols):
    rng = np.random.default_rng(cols)
    rows = 24
    rb = oracle.planar_row_bytes(cols)
    planar = rng.integers(0, 256, rows * rb, dtype=np.uint8)  # junk bytes (27, 55, ..., 251..255) decode to zero trits
    planar[: min(256, planar.size)] = np.arange(min(256, planar.size), dtype=np.uint8)
    ws = (0.5 + rng.random(rows * cols // 64)).astype(np.float16).astype(np.float32)
    acts = rng.integers(-128, 128, cols, dtype=np.int8)
    acts[:4] = [-128, -128, 127, 127]
    sc = rng.random(cols // 32).astype(np.float32)
    a, b, _ = _both(oracle, lambda: oracle.gemv_block_scaled(planar, ws, acts, sc, rows, cols))
    assert np.array_equal(_bits(a), _bits(b))


@pytest.mark.parametrize("arch,f32_values,bf16", [(0, False, False), (0, True, False), (1, False, True)])
def test_whole_token_logits(oracle, arch, f32_values, bf16):
    spec = synth.make_model(arch, f32_values, 256, 512, 2, 4, 2, 64, 300, 256, 500000.0, 1e-5, config=5, random_norms=True, bf16_tables=bf16)

    def run():
        m = oracle.Model(spec)
        return np.stack([m.forward(int(t), p) for p, t in enumerate(synth.prompt_tokens(5, 6, spec["vocab"]))])

    a, b, fast = _both(oracle, run)
    assert np.array_equal(_bits(a), _bits(b))
    if not fast:
        pytest.skip("this CPU has no AVX2 + FMA + F16C: only the portable loops ran")
