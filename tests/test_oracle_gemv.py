"""Pins the oracle's exact GEMV and activation quantiser.

The reference's rule (README.md:103, CONTRIBUTING.md:55-64): every kernel equals a brute-force i64 product. The
pattern grid is the one of rust/crates/quintrit-cuda/tests/gemv.rs:77-104 (weights +1 / -1 / 0 / random, activations
127 / -128 / alternating / random, nine column counts); the constant patterns have closed-form answers. Quantiser
known answers: rust/crates/quintrit-runtime/src/ops.rs:1968-1992.
"""
import numpy as np
import pytest

COLS = [1, 160, 161, 320, 2560, 3072, 4096, 13312, 23040]


def _weights(kind, n, rng):
    return {"random": lambda: rng.integers(-1, 2, n), "plus": lambda: np.ones(n), "minus": lambda: -np.ones(n),
            "zero": lambda: np.zeros(n)}[kind]().astype(np.int8)


def _acts(kind, n, rng):
    if kind == "random":
        return rng.integers(-128, 128, n).astype(np.int8)
    if kind == "max":
        return np.full(n, 127, np.int8)
    if kind == "min":
        return np.full(n, -128, np.int8)
    return np.where(np.arange(n) % 2 == 0, 127, -128).astype(np.int8)


@pytest.mark.parametrize("cols", COLS)
def test_every_gemv_path_equals_brute_force_on_the_reference_pattern_grid(oracle, cols):
    rng = np.random.default_rng(7 + cols)
    rows = 64
    for wk in ["random", "plus", "minus", "zero"]:
        trits = _weights(wk, rows * cols, rng)
        planar = oracle.pack_planar(trits, rows, cols)
        tiled = oracle.tile32(planar, rows, cols)
        tiled64 = oracle.tile64(planar, rows, cols)
        for ak in ["random", "max", "min", "alternating"]:
            act = _acts(ak, cols, rng)
            want = oracle.gemv_bruteforce(trits, rows, cols, act)
            # closed forms for the constant patterns
            if wk in ("plus", "minus"):
                assert np.all(want == (1 if wk == "plus" else -1) * int(act.astype(np.int64).sum()))
            if wk == "zero":
                assert np.all(want == 0)
            assert np.array_equal(oracle.gemv_planar(planar, rows, cols, act), want), (wk, ak)
            assert np.array_equal(oracle.gemv_lut_wide(tiled, rows, cols, act), want), (wk, ak)
            if oracle.cpu_has_avx512_vbmi():
                for threads in (1, 3):
                    assert np.array_equal(oracle.cpu_gemv_avx512(tiled64, rows, cols, act, threads), want), (wk, ak)
            assert np.array_equal(oracle.cpu_gemv_portable(planar, rows, cols, act, 2), want)


def test_awkward_row_counts_on_the_timed_kernel(oracle):
    # quintrit-cuda/tests/gemv.rs:110-126 row counts; the 64-row tiling pads with zero weights
    if not oracle.cpu_has_avx512_vbmi():
        pytest.skip("no AVX-512 VBMI on this host")
    rng = np.random.default_rng(11)
    for rows, cols in [(2, 160), (6, 3072), (12, 2560), (40, 3072), (200, 321)]:
        trits = rng.integers(-1, 2, rows * cols).astype(np.int8)
        act = rng.integers(-128, 128, cols).astype(np.int8)
        planar = oracle.pack_planar(trits, rows, cols)
        got = oracle.cpu_gemv_avx512(oracle.tile64(planar, rows, cols), rows, cols, act, 4)
        assert np.array_equal(got, oracle.gemv_bruteforce(trits, rows, cols, act))


def test_quantiser_known_answers(oracle):
    q, s = oracle.quantize_int8([0.5, -1.0, 0.25, 1.0, -0.001])
    assert s == np.float32(127.0) and list(q) == [64, -127, 32, 127, 0]
    q, s = oracle.quantize_int8(np.zeros(8))
    assert s == 0.0 and not q.any()


def test_quantiser_rounds_half_away_and_clamps(oracle):
    # ops.rs:258-263: round() is half away from zero; codes are clamped to [-128, 127]
    x = np.array([127.0, 0.5, -0.5, 1.5, -1.5, 2.5, -127.0], np.float32)
    q, s = oracle.quantize_int8(x)
    assert s == 1.0 and list(q) == [127, 1, -1, 2, -2, 3, -127]
    rng = np.random.default_rng(3)
    x = rng.standard_normal(3072).astype(np.float32)
    q, s = oracle.quantize_int8(x)
    y = x * s
    want = np.clip(np.sign(y) * np.floor(np.abs(y) + np.float32(0.5)), -128, 127).astype(np.int8)
    assert np.array_equal(q, want) and np.abs(q).max() == 127


def test_rescale_is_one_division_and_one_multiply(oracle):
    # quintrit-runtime/src/layer.rs:143-150
    acc = np.array([5, -7, 0, 123456], np.int32)
    ws, s = np.float32(0.37), np.float32(41.3)
    assert np.array_equal(oracle.rescale(acc, ws, s), acc.astype(np.float32) * np.float32(ws / s))
    assert not oracle.rescale(acc, ws, 0.0).any()
