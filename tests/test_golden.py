"""The committed fixture tests/golden/golden.npz (made by tests/golden/make_golden.py from seeded inputs): the CPU oracle must
still reproduce it (CPU test), and the CUDA path must reproduce it through the C ABI (GPU test). The fixture also carries
known answers of the reference's own unit tests, which the oracle is checked against here once more."""
import os

import numpy as np
import pytest

import quintrit_b200 as q
from quintrit_b200 import gguf_io

HERE = os.path.dirname(os.path.abspath(__file__))
GEMV_SHAPES = [(33, 161), (64, 320), (96, 3072), (40, 23040)]


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(HERE, "golden", "golden.npz"))


def _spec(arch, f32v):
    import importlib.util

    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.model_spec(arch, f32v)


def test_oracle_reproduces_the_fixture(oracle, gold):
    for i, (rows, cols) in enumerate(GEMV_SHAPES):
        assert np.array_equal(oracle.gemv_planar(gold[f"gemv{i}_planar"], rows, cols, gold[f"gemv{i}_act"]), gold[f"gemv{i}_out"])
    codes, scale = oracle.quantize_int8(gold["ref_quant_in"])
    assert np.array_equal(codes, gold["ref_quant_codes"]) and np.float32(scale) == gold["ref_quant_scale"][0]
    assert [oracle.planar_row_bytes(int(c)) for c in gold["ref_row_bytes_cols"]] == list(gold["ref_row_bytes"])
    qs, d = oracle.quantize_q8_0(gold["bs_x"])
    assert np.array_equal(qs, gold["bs_codes"]) and np.array_equal(d.view(np.uint32), gold["bs_scales"].view(np.uint32))
    planar = oracle.pack_planar(gold["bs_trits"].reshape(-1), 17, 640)
    assert np.array_equal(oracle.gemv_block_scaled(planar, gold["bs_wscales"], qs, d, 17, 640).view(np.uint32), gold["bs_out_bits"])
    spec = _spec(0, False)
    ref = oracle.Model(spec)
    want = gold["model_a0_f0_logits_bits"]
    for p, t in enumerate(gold["model_a0_f0_tokens"][:3]):
        assert np.array_equal(ref.forward(int(t), p).view(np.uint32), want[p])


@pytest.mark.gpu
def test_cuda_path_reproduces_the_fixture(gold):
    for i, (rows, cols) in enumerate(GEMV_SHAPES):
        m = q.Matrix(gold[f"gemv{i}_planar"], rows, cols)
        assert np.array_equal(m.gemv_i32(gold[f"gemv{i}_act"]), gold[f"gemv{i}_out"])
        m.free()
    sc16 = gold["bs_wscales"].astype(np.float16)
    m = q.Matrix(gguf_io.encode_q2_0(gold["bs_trits"], sc16), 17, 640, q.SRC_Q2_0)
    assert np.array_equal(m.gemv_block_scaled(gold["bs_x"]).view(np.uint32), gold["bs_out_bits"])
    m.free()
    for arch in (0, 1):
        for f32v in (False, True):
            dec = q.Decoder(_spec(arch, f32v))
            want = gold[f"model_a{arch}_f{int(f32v)}_logits_bits"]
            for p, t in enumerate(gold[f"model_a{arch}_f{int(f32v)}_tokens"]):
                got, _ = dec.forward(int(t), p)
                assert np.array_equal(got.view(np.uint32), want[p]), (arch, f32v, p)
            dec.free()
