"""Pins of the block-scaled (Q2_0 x Q8_0) oracle: the reference's own test grid and known answers.
rust/crates/quintrit-core/src/block_scaled.rs:1034-1135 (two formulations agree bit for bit on ten shapes),
rust/crates/quintrit-runtime/tests/model_ops_tests.rs:51-70 (Q8_0 quantiser properties)."""
import numpy as np
import pytest

import oracle

GRID = [(1, 64), (3, 128), (70, 192), (65, 320), (33, 2048), (130, 2560), (17, 640), (9, 704), (66, 1280), (5, 9728)]


def _case(rows, cols, seed):
    rng = np.random.default_rng(seed)
    trits = rng.integers(-1, 2, size=(rows, cols)).astype(np.int8)
    ws = (rng.integers(0, 1000, size=rows * cols // 64).astype(np.float32) * np.float32(1e-4) + np.float32(1e-3)).astype(np.float32)
    acts = rng.integers(-128, 127, size=cols).astype(np.int8)
    a_s = (rng.integers(0, 977, size=cols // 32).astype(np.float32) * np.float32(3e-3) + np.float32(1e-2)).astype(np.float32)
    return trits, ws, acts, a_s


@pytest.mark.parametrize("rows,cols", GRID)
def test_planar_and_trit_formulations_agree_bitwise(rows, cols):
    trits, ws, acts, a_s = _case(rows, cols, rows * 100003 + cols)
    planar = oracle.pack_planar(trits.reshape(-1), rows, cols)
    rb = oracle.planar_row_bytes(cols)
    got = oracle.gemv_block_scaled(planar, ws, acts, a_s, rows, cols)
    for r in range(rows):
        want = oracle.block_scaled_dot_trits(trits[r], ws[r * cols // 64:(r + 1) * cols // 64], acts, a_s, cols)
        one = oracle.block_scaled_dot_row(planar[r * rb:(r + 1) * rb], ws[r * cols // 64:(r + 1) * cols // 64], acts, a_s, cols)
        assert want.view(np.uint32) == one.view(np.uint32) == got[r:r + 1].view(np.uint32)[0], (r, rows, cols)


def test_block_scaled_closed_forms():
    # all weights +1, all codes 1, scales 1: every lane sum is 4, 8 lanes, cols/32 blocks -> the sum is exactly cols
    for cols in (64, 320, 704):
        trits = np.ones(cols, np.int8)
        ws, a_s = np.ones(cols // 64, np.float32), np.ones(cols // 32, np.float32)
        assert oracle.block_scaled_dot_trits(trits, ws, np.ones(cols, np.int8), a_s, cols) == np.float32(cols)
        # the scale of a 64-block multiplies both of its activation blocks
        ws2 = ws.copy()
        ws2[0] = 0.5
        assert oracle.block_scaled_dot_trits(trits, ws2, np.ones(cols, np.int8), a_s, cols) == np.float32(cols - 32)


def test_q8_0_quantiser_known_answers():
    rng = np.random.default_rng(2)
    x = (rng.uniform(-1, 1, 256) * (1 + np.arange(256) % 7)).astype(np.float32)
    qs, d = oracle.quantize_q8_0(x)
    for b in range(8):
        xb = x[b * 32:(b + 1) * 32]
        amax = np.abs(xb).max()
        assert abs(d[b] - amax / 127.0) <= amax / 127.0 * 1e-3
        assert (np.abs(qs[b * 32:(b + 1) * 32].astype(np.int32)) == 127).any()
        assert (np.abs(qs[b * 32:(b + 1) * 32].astype(np.float32) * d[b] - xb) <= 0.5 * d[b] + amax * 2e-3).all()
        # the definition itself: d = f16(amax / 127), q = round_ties_even(x * (127 / amax))
        want_d = np.float32(np.float16(np.float32(amax) / np.float32(127.0)))
        assert d[b] == want_d
        want_q = np.clip(np.rint(xb * (np.float32(127.0) / np.float32(amax))), -128, 127).astype(np.int8)
        assert np.array_equal(qs[b * 32:(b + 1) * 32], want_q)
    qz, dz = oracle.quantize_q8_0(np.zeros(32, np.float32))
    assert not qz.any() and dz[0] == 0.0
    # ties go to even, NaN gives 0 and is ignored by amax
    y = np.zeros(32, np.float32)
    y[0], y[1], y[2], y[3], y[4] = 127.0, 0.5, 1.5, 2.5, np.nan
    q, dd = oracle.quantize_q8_0(y)
    assert list(q[:5]) == [127, 0, 2, 2, 0] and dd[0] == 1.0
