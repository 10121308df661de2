"""Pins the oracle's GGUF ternary decoders to the known answers of the reference's tests.

Sources: rust/crates/quintrit-format/tests/gguf_decoder_tests.rs:430-597 (ggml layouts, encoders with ceiling-division
digit packing, uniform-scale bit patterns), rust/crates/quintrit-format/src/decoders/q2_0.rs:161-187,
rust/crates/quintrit-format/src/decoders/i2_s.rs:20-40, rust/crates/quintrit-py/tests/gguf_builder.py:80-86.
"""
import numpy as np
import pytest


from quintrit_b200.gguf_io import encode_tq1_0 as _enc1, encode_tq2_0 as _enc2


def encode_tq2_0(trits, d_bits=0x3800):
    return _enc2(trits, d_bits).reshape(-1, 66)


def encode_tq1_0(trits, d_bits=0x3800):
    return _enc1(trits, d_bits).reshape(-1, 54)


def _trits(n, seed):
    return np.random.default_rng(seed).integers(-1, 2, n).astype(np.int8)


@pytest.mark.parametrize("rows,cols", [(1, 256), (4, 256), (3, 512), (32, 1024)])
def test_tq_decoders_invert_the_encoders(oracle, rows, cols):
    t = _trits(rows * cols, 77 + rows)
    assert np.array_equal(oracle.decode_tq2_0(encode_tq2_0(t), rows, cols).reshape(-1), t)
    assert np.array_equal(oracle.decode_tq1_0(encode_tq1_0(t), rows, cols).reshape(-1), t)


@pytest.mark.parametrize("v", [-1, 0, 1])
def test_tq_extremes(oracle, v):
    t = np.full(256, v, np.int8)
    assert np.array_equal(oracle.decode_tq2_0(encode_tq2_0(t), 1, 256).reshape(-1), t)
    assert np.array_equal(oracle.decode_tq1_0(encode_tq1_0(t), 1, 256).reshape(-1), t)


def test_tq_layouts_on_arbitrary_bytes(oracle):
    # every byte value is defined for both decoders: digit n of a TQ1_0 byte is ((byte * 3^n mod 256) * 3) >> 8, minus 1
    block = ((np.arange(66) * 73 + 29) % 251).astype(np.uint8)
    got = oracle.decode_tq2_0(block, 1, 256).reshape(-1)
    want = []
    for j in (0, 32):
        for l in range(4):
            for m in range(32):
                code = (int(block[j + m]) >> (2 * l)) & 3
                want.append({0: -1, 2: 1}.get(code, 0))
    assert list(got) == want
    block = ((np.arange(54) * 73 + 29) % 251).astype(np.uint8)
    got = oracle.decode_tq1_0(block, 1, 256).reshape(-1)
    digit = lambda b, n: ((((int(b) * 3 ** n) & 0xFF) * 3) >> 8) - 1
    want = [digit(block[m], n) for n in range(5) for m in range(32)]
    want += [digit(block[32 + m], n) for n in range(5) for m in range(16)]
    want += [digit(block[48 + j], n) for n in range(4) for j in range(4)]
    assert list(got) == want


def test_uniform_block_scale_bit_patterns(oracle):
    t = _trits(4 * 256, 5)
    for ty, enc in ((34, encode_tq1_0), (35, encode_tq2_0)):
        assert oracle.uniform_block_scale(ty, enc(t, 0x3800)) == 0.5
        assert oracle.uniform_block_scale(ty, enc(t, 0x3C00)) == 1.0
        assert oracle.uniform_block_scale(ty, enc(t, 0xC000)) == -2.0
        assert oracle.uniform_block_scale(ty, enc(t, 0x0001)) == np.float32(2.0 ** -24)
        assert oracle.uniform_block_scale(ty, enc(t, 0x0000)) == 0.0
        mixed = enc(t, 0x3800)
        mixed[2, -2:] = (0x00, 0x3C)
        assert oracle.uniform_block_scale(ty, mixed) is None
    assert oracle.uniform_block_scale(36, np.zeros(66, np.uint8)) is None


def test_i2_s_layout(oracle):
    # i2_s.rs:20-40: code = trit + 1, element j of a 128-block goes to byte j % 32, bits 6 - 2 * (j / 32)
    rows, cols = 3, 384
    t = _trits(rows * cols, 9)
    data = oracle.encode_i2_s(t, rows, cols)
    # numpy twin of the packer
    codes = (t.reshape(rows, cols // 128, 4, 32) + 1).astype(np.uint8)
    want = (codes[:, :, 0] << 6) | (codes[:, :, 1] << 4) | (codes[:, :, 2] << 2) | codes[:, :, 3]
    assert np.array_equal(data, want.reshape(-1))
    assert np.array_equal(oracle.decode_i2_s(data, rows, cols).reshape(-1), t)
    # the unused code 3 decodes to zero (quintrit-core/src/unpack.rs:49-52)
    assert not oracle.decode_i2_s(np.full(32, 0xFF, np.uint8), 1, 128).any()
    with pytest.raises(ValueError):
        oracle.decode_i2_s(data, rows, cols + 1)


def test_q2_0_known_answers(oracle):
    # q2_0.rs:161-176
    codes = (np.arange(128) % 3).astype(np.uint8)
    pack = lambda c: (c[0::4] | (c[1::4] << 2) | (c[2::4] << 4) | (c[3::4] << 6)).astype(np.uint8)
    b64 = np.concatenate([[0x00, 0x3C], pack(codes[:64]), [0x00, 0x38], pack(codes[64:])]).astype(np.uint8)
    t, s = oracle.decode_q2_0(b64, 1, 128)
    assert list(s) == [1.0, 0.5]
    assert list(t.reshape(-1)[:6]) == [-1, 0, 1, -1, 0, 1]
    assert np.array_equal(t.reshape(-1), codes.astype(np.int8) - 1)
    # q2_0.rs:178-186
    bad = np.concatenate([[0x00, 0x3C], np.full(16, 3)]).astype(np.uint8)
    for rows, cols in [(1, 64), (1, 96), (2, 64)]:
        with pytest.raises(ValueError):
            oracle.decode_q2_0(bad, rows, cols)


def test_half_to_f32_is_exact_for_every_half(oracle):
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([oracle.half_to_f32(int(x)) for x in h[::7]], np.float32)
    w = want[::7]
    same = (got.view(np.uint32) == w.view(np.uint32)) | (np.isnan(got) & np.isnan(w))
    assert same.all()
