"""Pins the oracle's velurex byte and planar layout to the known answers of the reference's own tests.

Sources: rust/crates/quintrit-core/tests/pack_tests.rs:8-53, 103-130; docs/velurex-encoding.md:21-34;
rust/crates/quintrit-cuda/src/pack.rs:103-149; docs/simd-decode.md:35-58.
"""
import itertools

import numpy as np


def test_all_243_states_roundtrip_and_stay_below_251(oracle):
    # pack_tests.rs:8-40
    seen = set()
    for d in itertools.product(range(3), repeat=5):
        t = [x - 1 for x in d]
        b = oracle.pack_5trits(t)
        assert b == d[0] + 3 * d[1] + 9 * d[2] + 28 * d[3] + 84 * d[4]
        assert b <= 250
        assert list(oracle.byte_to_trits(b)) == t
        seen.add(b)
    assert len(seen) == 243
    assert max(seen) == 250 and min(seen) == 0
    # velurex-encoding.md:34: one gap after every 27 values
    for gap in (27, 55, 83, 111, 139, 167, 195, 223):
        assert gap not in seen


def test_unused_bytes_decode_to_zero(oracle):
    # pack_tests.rs:43-53 (251..255) and the in-range gaps, which the table never assigns either
    for b in list(range(251, 256)) + [27, 55, 83, 111, 139, 167, 195, 223]:
        assert list(oracle.byte_to_trits(b)) == [0, 0, 0, 0, 0]


def test_division_free_identities_hold_for_every_valid_byte(oracle):
    # simd-decode.md:35-58 and quintrit-cuda/kernels/gemv.cu:14 ((b * 781) >> 16 == b / 84)
    for b in range(251):
        v11 = b >> 2
        v15 = b >> 5
        v17 = (v11 + v15 + 1) >> 1
        assert v17 >> 2 == b // 28
        assert (b * 781) >> 16 == b // 84


def test_row_sizes(oracle):
    # quintrit-cuda/src/pack.rs:142-149 and core/pack.rs:218-227 (3072 columns: rows of 616 bytes in a tile)
    assert oracle.planar_row_bytes(3072) == 640
    assert oracle.planar_row_bytes(23040) == 4608
    assert oracle.planar_row_bytes(160) == 32
    assert oracle.planar_row_bytes(161) == 64
    assert oracle.tile_row_bytes(3072) == 616
    assert oracle.tile_row_bytes(160) == 32
    assert oracle.tile_row_bytes(1) == 2


def _lcg_trits(n, seed):
    # quintrit-cuda/src/pack.rs:124-131
    out = np.empty(n, np.int8)
    s = seed
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = (s >> 33) % 3 - 1
    return out


def _pack_by_definition(trits, rows, cols):
    # the layout as stated in quintrit-cuda/src/pack.rs:3-6, written out with numpy
    bpr = -(-cols // 160)
    padded = np.zeros((rows, bpr * 160), np.int64)
    padded[:, :cols] = trits.reshape(rows, cols)
    d = padded.reshape(rows, bpr, 5, 32) + 1
    radix = np.array([1, 3, 9, 28, 84]).reshape(1, 1, 5, 1)
    return (d * radix).sum(axis=2).astype(np.uint8).reshape(-1)


def test_planar_layout_matches_its_definition(oracle):
    # quintrit-cuda/src/pack.rs:134-140
    for rows, cols in [(1, 1), (3, 160), (4, 161), (5, 3072), (2, 2560), (2, 319)]:
        trits = _lcg_trits(rows * cols, rows * 31 + cols)
        got = oracle.pack_planar(trits, rows, cols)
        assert np.array_equal(got, _pack_by_definition(trits, rows, cols)), (rows, cols)
        assert np.array_equal(oracle.unpack_planar(got, rows, cols).reshape(-1), trits)


def test_matrix_roundtrip_shapes(oracle):
    # pack_tests.rs:55-80
    for rows, cols in [(32, 160), (32, 320), (64, 640), (128, 1600), (1, 160)]:
        trits = ((np.arange(rows * cols) * 7 + 1) % 3 - 1).astype(np.int8)
        packed = oracle.pack_planar(trits, rows, cols)
        assert np.array_equal(oracle.unpack_planar(packed, rows, cols).reshape(-1), trits)


def test_tile_layout_keeps_every_product(oracle):
    # pack_tests.rs:103-130 checks the tile transform is lossless for every tail length; here the equivalent statement:
    # the activation a tile byte multiplies (column_activation_index) reproduces the brute-force product.
    rng = np.random.default_rng(5)
    for cols in [1, 5, 31, 32, 33, 159, 160, 161, 192, 250, 320, 321, 479, 800, 3079]:
        rows = 32
        trits = rng.integers(-1, 2, rows * cols).astype(np.int8)
        act = rng.integers(-128, 128, cols).astype(np.int8)
        tiled = oracle.tile32(oracle.pack_planar(trits, rows, cols), rows, cols)
        rb = oracle.tile_row_bytes(cols)
        assert tiled.size == rows * rb
        want = oracle.gemv_bruteforce(trits, rows, cols, act)
        got = np.zeros(rows, np.int64)
        for c in range(rb):
            for r in range(rows):
                t = oracle.byte_to_trits(int(tiled[c * 32 + r]))
                for p in range(5):
                    idx = oracle.column_activation_index(cols, c, p)
                    if idx < cols:
                        got[r] += int(t[p]) * int(act[idx])
        assert np.array_equal(got, want), cols
