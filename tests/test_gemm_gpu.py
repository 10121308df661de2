"""The batched projection on the tensor cores (tcgen05 int8, quintrit_b200_gemm_i32) against the batch-1 kernel and the CPU oracle: a batch of
B activation vectors gives, vector by vector, the integers of B single projections (the reference runs a prompt token by token,
quintrit-runtime/src/gpu.rs:459-493; a batched path must not change a bit of it)."""
import numpy as np
import pytest

import oracle
import quintrit_b200 as q

pytestmark = pytest.mark.gpu


def _case(rows, cols, batch, seed):
    rng = np.random.default_rng(seed)
    trits = rng.integers(-1, 2, size=(rows, cols)).astype(np.int8)
    acts = rng.integers(-128, 128, size=(batch, cols)).astype(np.int8)
    return trits, acts


@pytest.mark.parametrize("rows,cols,batch", [(128, 160, 16), (96, 161, 1), (200, 333, 37), (1024, 3072, 128), (3072, 3072, 64), (256, 23040, 48), (2304, 3072, 256)])
def test_batched_projection_equals_single_projections(rows, cols, batch):
    trits, acts = _case(rows, cols, batch, rows + cols + batch)
    m = q.Matrix.from_trits(trits, rows, cols)
    got = m.gemm_i32(acts)
    assert got.shape == (batch, rows)
    want = acts.astype(np.int64) @ trits.astype(np.int64).T
    assert np.array_equal(got, want)
    for b in (0, batch - 1):
        assert np.array_equal(got[b], m.gemv_i32(acts[b]))
    assert np.array_equal(got[0], oracle.gemv_bruteforce(trits, rows, cols, acts[0]))


def test_extreme_activations_and_long_batches():
    rows, cols = 384, 2560
    trits, _ = _case(rows, cols, 1, 9)
    m = q.Matrix.from_trits(trits, rows, cols)
    acts = np.stack([np.full(cols, 127, np.int8), np.full(cols, -128, np.int8), np.zeros(cols, np.int8), np.where(np.arange(cols) % 2 == 0, 127, -128).astype(np.int8)])
    assert np.array_equal(m.gemm_i32(acts), acts.astype(np.int64) @ trits.astype(np.int64).T)
    # all +1 weights against 127: the largest sum a row can hold
    ones = q.Matrix.from_trits(np.ones((128, cols), np.int8), 128, cols)
    assert (ones.gemm_i32(acts[:1]) == 127 * cols).all()
    # more vectors than one launch takes (256): several launches behind one call
    rng = np.random.default_rng(10)
    many = rng.integers(-128, 128, size=(700, cols)).astype(np.int8)
    assert np.array_equal(m.gemm_i32(many), many.astype(np.int64) @ trits.astype(np.int64).T)


def test_arguments():
    m = q.Matrix.from_trits(np.zeros((64, 160), np.int8), 64, 160)
    lib = q.load_library()
    out = np.zeros(64, np.int32)
    act = np.zeros(160, np.int8)
    import ctypes as C

    i8p, i32p = C.POINTER(C.c_int8), C.POINTER(C.c_int32)
    assert lib.quintrit_b200_gemm_i32(m.handle, act.ctypes.data_as(i8p), 160, 0, out.ctypes.data_as(i32p), 64) == 2
    assert lib.quintrit_b200_gemm_i32(m.handle, act.ctypes.data_as(i8p), 100, 1, out.ctypes.data_as(i32p), 64) == 4
    assert lib.quintrit_b200_gemm_i32(m.handle, act.ctypes.data_as(i8p), 160, 1, out.ctypes.data_as(i32p), 10) == 4
    assert lib.quintrit_b200_gemm_i32(m.handle, None, 160, 1, out.ctypes.data_as(i32p), 64) == 1
    assert lib.quintrit_b200_gemm_i32(None, act.ctypes.data_as(i8p), 160, 1, out.ctypes.data_as(i32p), 64) == 14
