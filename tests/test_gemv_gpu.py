"""GPU parity of the velurex GEMV through the C ABI against the CPU oracle: bit-exact int32.

Mirrors rust/crates/quintrit-cuda/tests/gemv.rs:77-139 (pattern grid, awkward row counts, invalid launches).
"""
import ctypes as C

import numpy as np
import pytest

import quintrit_b200 as q

pytestmark = pytest.mark.gpu

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


def test_device_is_a_supported_b200():
    assert q.device_count() >= 1
    info = q.device_info(0)
    assert info.supported and info.compute_major == 10 and info.sm_count > 0


@pytest.mark.parametrize("cols", COLS)
def test_projection_is_exact_for_every_shape_and_pattern(oracle, cols):
    rng = np.random.default_rng(7 + cols)
    rows = 64
    for wk in ["random", "plus", "minus", "zero"]:
        trits = _weights(wk, rows * cols, rng)
        m = q.Matrix.from_trits(trits, rows, cols)
        for ak in ["random", "max", "min", "alternating"]:
            act = _acts(ak, cols, rng)
            want = oracle.gemv_bruteforce(trits, rows, cols, act)
            got = m.gemv_i32(act)
            assert np.array_equal(got.astype(np.int64), want), (cols, wk, ak)
        m.free()


@pytest.mark.parametrize("rows,cols", [(2, 160), (6, 3072), (12, 2560), (40, 3072), (2560, 2560), (3456, 2560), (33, 161), (1, 1), (1000, 23040)])
def test_awkward_row_counts(oracle, rows, cols):
    rng = np.random.default_rng(11 + rows)
    trits = rng.integers(-1, 2, rows * cols).astype(np.int8)
    act = rng.integers(-128, 128, cols).astype(np.int8)
    planar = oracle.pack_planar(trits, rows, cols)
    m = q.Matrix(planar, rows, cols)
    assert np.array_equal(m.gemv_i32(act), oracle.gemv_planar(planar, rows, cols, act))
    # the call can be repeated: the work counters re-arm themselves
    act2 = rng.integers(-128, 128, cols).astype(np.int8)
    assert np.array_equal(m.gemv_i32(act2), oracle.gemv_planar(planar, rows, cols, act2))


def test_device_layout_round_trips_to_the_reference_planar_bytes(oracle):
    rng = np.random.default_rng(3)
    for rows, cols in [(1, 1), (5, 159), (32, 160), (33, 161), (70, 3072), (64, 3079)]:
        trits = rng.integers(-1, 2, rows * cols).astype(np.int8)
        planar = oracle.pack_planar(trits, rows, cols)
        m = q.Matrix(planar, rows, cols)
        assert np.array_equal(m.download_planar(), planar), (rows, cols)
        assert m.device_bytes == -(-cols // 160) * -(-rows // 32) * 1024


def test_rescaled_output_matches_the_layer_forward(oracle):
    rng = np.random.default_rng(5)
    rows, cols = 3072, 3072
    trits = rng.choice([-1, 1, 0], rows * cols, p=[0.3, 0.3, 0.4]).astype(np.int8)
    x = rng.standard_normal(cols).astype(np.float32)
    act, s = oracle.quantize_int8(x)
    ws = np.float32(1.37)
    m = q.Matrix.from_trits(trits, rows, cols)
    acc = m.gemv_i32(act)
    assert np.array_equal(acc.astype(np.int64), oracle.gemv_bruteforce(trits, rows, cols, act))
    got = m.forward(act, s, ws)
    assert np.array_equal(got.view(np.uint32), oracle.rescale(acc, ws, s).view(np.uint32))
    assert not m.forward(act, 0.0, ws).any()


def test_invalid_calls_are_rejected():
    rng = np.random.default_rng(2)
    m = q.Matrix.from_trits(rng.integers(-1, 2, 8 * 160).astype(np.int8), 8, 160)
    with pytest.raises(q.QuintritError) as e:
        m.gemv_i32(np.zeros(100, np.int8))  # too few activations
    assert e.value.code == 4
    lib = q.load_library()
    out = np.zeros(4, np.int32)
    a = np.zeros(160, np.int8)
    rc = lib.quintrit_b200_gemv_i32(m.handle, a.ctypes.data_as(C.POINTER(C.c_int8)), 160, out.ctypes.data_as(C.POINTER(C.c_int32)), 4)
    assert rc == 4
    with pytest.raises(q.QuintritError):
        q.Matrix(np.zeros(10, np.uint8), 8, 160)  # payload too short
    m.free()
    assert lib.quintrit_b200_gemv_i32(m.handle, a.ctypes.data_as(C.POINTER(C.c_int8)), 160, out.ctypes.data_as(C.POINTER(C.c_int32)), 4) == 14


def test_gguf_sources_transcode_on_device(oracle):
    from tests.test_oracle_decoders import encode_tq1_0, encode_tq2_0

    rng = np.random.default_rng(9)
    rows, cols = 96, 768
    trits = rng.integers(-1, 2, rows * cols).astype(np.int8)
    planar = oracle.pack_planar(trits, rows, cols)
    act = rng.integers(-128, 128, cols).astype(np.int8)
    want = oracle.gemv_bruteforce(trits, rows, cols, act)
    for src, data in [(q.SRC_I2_S, oracle.encode_i2_s(trits, rows, cols)), (q.SRC_TQ2_0, encode_tq2_0(trits)), (q.SRC_TQ1_0, encode_tq1_0(trits))]:
        m = q.Matrix(data, rows, cols, source=src)
        assert np.array_equal(m.download_planar(), planar), src
        assert np.array_equal(m.gemv_i32(act).astype(np.int64), want), src


@pytest.mark.parametrize("segments", [None, 3, 16])
def test_plan_runs_many_projections_in_one_launch(oracle, monkeypatch, segments):
    """A plan's host-buffer run is one launch for a small plan; large plans (and this test, through the experiment knob) run in segments of
    consecutive matrices whose copies overlap the other segments' kernels: the results are the same."""
    if segments is not None:
        monkeypatch.setenv("QUINTRIT_B200_PLAN_SEGMENTS", str(segments))
    rng = np.random.default_rng(13)
    shapes = [(3072, 3072), (1024, 3072), (1024, 3072), (3072, 3072), (2304, 3072), (2304, 3072), (3072, 2304), (40, 161), (7, 1)]
    mats, planars, acts = [], [], []
    for rows, cols in shapes:
        trits = rng.choice([-1, 1, 0], rows * cols, p=[0.3, 0.3, 0.4]).astype(np.int8)
        planars.append(oracle.pack_planar(trits, rows, cols))
        mats.append(q.Matrix(planars[-1], rows, cols))
        acts.append(rng.integers(-128, 128, cols).astype(np.int8))
    plan = q.Plan(mats)
    for _ in range(2):
        q.launch_count(reset=True)
        res = plan.split_results(plan.run(plan.pack_activations(acts)))
        assert q.launch_count() == (1 if segments is None else min(segments, len(shapes)))
        for (rows, cols), planar, a, r in zip(shapes, planars, acts, res):
            assert np.array_equal(r, oracle.gemv_planar(planar, rows, cols, a)), (rows, cols)
        acts = [rng.integers(-128, 128, c).astype(np.int8) for _, c in shapes]
