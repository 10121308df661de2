"""GPU parity of the block-scaled (Q2_0 x Q8_0) path through the C ABI against the CPU oracle: on-device transcode of a
Q2_0 payload (planar bytes and per-64 scales bit-identical), the Q8_0 quantiser, and the GEMV whose floats must equal the
oracle's bit for bit on the shape grid of rust/crates/quintrit-core/src/block_scaled.rs:1051-1063 and on the model's
projection shapes. Error behaviour follows quintrit-format/src/decoders/q2_0.rs:17-55."""
import numpy as np
import pytest

import oracle
import quintrit_b200 as q

pytestmark = pytest.mark.gpu

GRID = [(1, 64), (3, 128), (70, 192), (65, 320), (33, 2048), (130, 2560), (17, 640), (9, 704), (66, 1280), (5, 9728), (256, 3072), (96, 23040),
        (9607, 192), (19001, 64), (3, 131072), (40, 49152)]  # more row groups than resident blocks; the widest rows (two ring slots); twelve slots


def q2_0_payload(trits: np.ndarray, scales_f16: np.ndarray) -> np.ndarray:
    """Q2_0 blocks of 64 weights: f16 scale, then 16 bytes of 2-bit codes (code = trit + 1), lowest bits first."""
    rows, cols = trits.shape
    codes = (trits.astype(np.int16) + 1).astype(np.uint8).reshape(rows * cols // 64, 16, 4)
    packed = codes[:, :, 0] | (codes[:, :, 1] << 2) | (codes[:, :, 2] << 4) | (codes[:, :, 3] << 6)
    out = np.zeros((rows * cols // 64, 18), np.uint8)
    out[:, :2] = scales_f16.reshape(-1).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = packed
    return out.reshape(-1)


def _case(rows, cols, seed):
    rng = np.random.default_rng(seed)
    trits = rng.integers(-1, 2, size=(rows, cols)).astype(np.int8)
    scales = rng.uniform(0.5, 2.0, size=rows * cols // 64).astype(np.float16)
    x = (rng.standard_normal(cols) * rng.uniform(0.1, 4.0)).astype(np.float32)
    return trits, scales, x


@pytest.mark.parametrize("rows,cols", GRID)
def test_transcode_and_gemv_equal_the_oracle_bitwise(rows, cols):
    trits, scales, x = _case(rows, cols, rows * 7919 + cols)
    payload = q2_0_payload(trits, scales)
    want_trits, want_scales = oracle.decode_q2_0(payload, rows, cols)
    assert np.array_equal(want_trits.reshape(rows, cols), trits)
    m = q.Matrix(payload, rows, cols, q.SRC_Q2_0)
    planar = oracle.pack_planar(trits.reshape(-1), rows, cols)
    assert np.array_equal(m.download_planar(), planar)
    assert np.array_equal(m.scales().view(np.uint32), np.asarray(want_scales, np.float32).view(np.uint32))
    qs, d = oracle.quantize_q8_0(x)
    gq, gd = q.quantize_q8_0(x)
    assert np.array_equal(gq, qs) and np.array_equal(gd.view(np.uint32), d.view(np.uint32))
    want = oracle.gemv_block_scaled(planar, want_scales, qs, d, rows, cols)
    got = m.gemv_block_scaled(x)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    got_q8 = m.gemv_block_scaled_q8(qs, d)
    assert np.array_equal(got_q8.view(np.uint32), want.view(np.uint32))
    m.free()


def test_quantiser_edge_values():
    y = np.zeros(64, np.float32)
    y[0], y[1], y[2], y[3], y[4] = 127.0, 0.5, 1.5, 2.5, np.nan
    want_q, want_d = oracle.quantize_q8_0(y)
    got_q, got_d = q.quantize_q8_0(y)
    assert np.array_equal(got_q, want_q) and np.array_equal(got_d.view(np.uint32), want_d.view(np.uint32))
    assert list(got_q[:5]) == [127, 0, 2, 2, 0] and got_d[1] == 0.0 and not got_q[32:].any()
    with pytest.raises(q.QuintritError) as e:
        q.quantize_q8_0(np.zeros(33, np.float32))
    assert e.value.code == 3  # QUINTRIT_ERR_INVALID_SHAPE


def test_rejections():
    trits, scales, _ = _case(4, 128, 5)
    payload = q2_0_payload(trits, scales)
    bad = payload.copy()
    bad[18 + 2 + 3] |= 0x0C  # second block, code byte 3: weight 64 + 13 gets the code 3
    with pytest.raises(q.QuintritError) as e:
        q.Matrix(bad, 4, 128, q.SRC_Q2_0)
    assert e.value.code == 8 and "77" in str(e.value) and "code 3" in str(e.value)  # QUINTRIT_ERR_FORMAT, first offending weight
    with pytest.raises(q.QuintritError) as e:
        q.Matrix(payload, 4, 96, q.SRC_Q2_0)  # not a multiple of 64
    assert e.value.code == 8
    m = q.Matrix(payload, 4, 128, q.SRC_Q2_0)
    with pytest.raises(q.QuintritError) as e:
        m.gemv_i32(np.zeros(128, np.int8))  # the integer GEMV does not serve block-scaled matrices
    assert e.value.code == 6
    with pytest.raises(q.QuintritError) as e:
        m.gemv_block_scaled(np.zeros(64, np.float32))
    assert e.value.code == 3
    plain = q.Matrix.from_trits(trits.reshape(-1), 4, 128)
    with pytest.raises(q.QuintritError) as e:
        plain.gemv_block_scaled(np.zeros(128, np.float32))
    assert e.value.code == 6
    m.free()
    plain.free()
