"""The reference's OWN CUDA kernels, compiled for sm_100a from the reference tree (oracle/_ref/libqtref_cuda.so, see oracle/refcuda.py), against the CPU
oracle and against the library, bit for bit. The reference asserts that these kernels equal its CPU runtime bitwise (quintrit-cuda/kernels/layer.cu:1-9,
quintrit-runtime/tests/gpu_layers.rs), so agreement here pins the oracle's restatement of the CPU runtime to code of the reference that runs on this machine."""
import numpy as np
import pytest

import oracle
import quintrit_b200 as q
from oracle import refcuda

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not refcuda.available(), reason="oracle/_ref/libqtref_cuda.so was not built (needs the reference tree at build time)")]


def _trits(rng, rows, cols):
    return rng.integers(-1, 2, size=(rows, cols)).astype(np.int8)


@pytest.mark.parametrize("cols", [160, 161, 333, 2560, 3072, 6912])
def test_gemv_of_every_reference_configuration(cols):
    rng = np.random.default_rng(cols)
    rows = 96
    trits = _trits(rng, rows, cols)
    planar = oracle.pack_planar(trits, rows, cols)
    mine = q.Matrix(planar, rows, cols)
    for act in (rng.integers(-128, 128, cols).astype(np.int8), np.full(cols, 127, np.int8), np.full(cols, -128, np.int8)):
        want = oracle.gemv_bruteforce(trits, rows, cols, act)
        for cfg, tag, per_block in refcuda.configs():
            assert rows % per_block == 0
            got = refcuda.gemv_plain(cfg, planar, rows, cols, act)
            assert np.array_equal(got, want), tag
        assert np.array_equal(mine.gemv_i32(act), want)


@pytest.mark.parametrize("activation", [0, 1])
def test_gated_epilogue(activation):
    rng = np.random.default_rng(11 + activation)
    n, cols = 256, 2560
    gate, up = _trits(rng, n, cols), _trits(rng, n, cols)
    inter = np.empty((2 * n, cols), np.int8)
    inter[0::2], inter[1::2] = gate, up
    x = rng.normal(0, 1, cols).astype(np.float32)
    act, s = oracle.quantize_int8(x)
    wsg, wsu = np.float32(0.037), np.float32(0.051)
    g = oracle.rescale(oracle.gemv_bruteforce(gate, n, cols, act), wsg, s)
    u = oracle.rescale(oracle.gemv_bruteforce(up, n, cols, act), wsu, s)
    want = oracle.swiglu(g, u) if activation == 0 else oracle.relu2_mul(g, u)
    for cfg in (0, 3):
        v, amax = refcuda.gemv_gated(cfg, oracle.pack_planar(inter, 2 * n, cols), 2 * n, cols, act, s, wsg, wsu, activation)
        assert np.array_equal(v.view(np.uint32), want.view(np.uint32))
        assert amax == np.abs(want).max()


@pytest.mark.parametrize("cols", [128, 2560, 3072, 6912])
def test_rms_norm_and_int8_quantiser(cols):
    rng = np.random.default_rng(cols + 1)
    x, gamma = rng.normal(0, 3, cols).astype(np.float32), rng.uniform(0.5, 1.5, cols).astype(np.float32)
    y = oracle.rms_norm(x, gamma, 1e-5)
    want_q, want_s = oracle.quantize_int8(y)
    got_q, got_s, total = refcuda.rms_quant(x, gamma, 1e-5, norm=True)
    assert got_s == want_s and np.array_equal(got_q, want_q) and total == int(want_q.astype(np.int64).sum())
    want_q, want_s = oracle.quantize_int8(x)  # without the norm: the quantiser alone
    got_q, got_s, _ = refcuda.rms_quant(x, gamma, 1e-5, norm=False)
    assert got_s == want_s and np.array_equal(got_q, want_q)
    zq, zs, _ = refcuda.rms_quant(np.zeros(cols, np.float32), gamma, 1e-5, norm=False)
    assert zs == 0 and not zq.any()


def test_output_head():
    rng = np.random.default_rng(3)
    vocab, cols = 1000, 2560
    h, w = rng.normal(0, 2, cols).astype(np.float32), rng.uniform(0.5, 1.5, cols).astype(np.float32)
    W = rng.normal(0, 0.02, (vocab, cols)).astype(np.float16).view(np.uint16)
    x16 = oracle.f32_to_f16_bits(oracle.rms_norm(h, w, 1e-5))
    normed, logits = refcuda.head(h, w, W, vocab, 1e-5)
    assert np.array_equal(normed.astype(np.float16).view(np.uint16), x16) and np.array_equal(normed, x16.view(np.float16).astype(np.float32))
    want = np.array([oracle.vec_dot_f16(x16, W[r]) for r in range(vocab)], np.float32)
    assert np.array_equal(logits.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("neox", [0, 1])
def test_rotary_embedding_and_kv_append(neox):
    rng = np.random.default_rng(5 + neox)
    q_heads, kv_heads, hd, pos = 4, 2, 128, 37
    qkv = rng.integers(-30000, 30000, (q_heads + 2 * kv_heads) * hd).astype(np.int32)
    s, wq, wk, wv = np.float32(17.3), np.float32(0.04), np.float32(0.05), np.float32(0.06)
    cos_sin = np.concatenate([oracle.rope_cache(p, hd, 500000.0) for p in range(pos + 1)])
    got_q, got_k, got_v = refcuda.rope_kv(qkv, s, wq, wk, wv, cos_sin, pos, q_heads, kv_heads, hd, hd, neox)
    nq, nk = q_heads * hd, kv_heads * hd
    cache = cos_sin[pos * hd:(pos + 1) * hd]
    want_q = oracle.rope_apply(oracle.rescale(qkv[:nq], wq, s), q_heads, hd, neox, cache)
    want_k = oracle.rope_apply(oracle.rescale(qkv[nq:nq + nk], wk, s), kv_heads, hd, neox, cache)
    want_v = oracle.rescale(qkv[nq + nk:], wv, s)
    assert np.array_equal(got_q.view(np.uint32), want_q.view(np.uint32))
    assert np.array_equal(got_k, oracle.f32_to_f16_bits(want_k)) and np.array_equal(got_v, oracle.f32_to_f16_bits(want_v))


@pytest.mark.parametrize("hd,cache_len,positions", [(128, 1024, [0, 6, 254, 255, 256, 300, 510, 511, 512, 700, 1023]), (256, 2048, [3, 511, 512, 1500, 2047]),
                                                    (64, 512, [100, 400, 511]), (32, 64, [0, 20, 63])])
def test_attention_with_the_f16_accumulator(hd, cache_len, positions):
    rng = np.random.default_rng(hd + cache_len)
    q_heads, kv_heads = 4, 2
    K = rng.normal(0, 1, (kv_heads, cache_len, hd)).astype(np.float16).view(np.uint16)
    V = rng.normal(0, 1, (kv_heads, cache_len, hd)).astype(np.float16).view(np.uint16)
    scale = np.float32(1.0 / np.sqrt(hd))
    for pos in positions:
        qv = rng.normal(0, 2, q_heads * hd).astype(np.float32)
        got = refcuda.attention(K, V, qv, q_heads, kv_heads, hd, cache_len, pos, scale)
        for h in range(q_heads):
            kvh = h // (q_heads // kv_heads)
            want = oracle.attend_head(qv[h * hd:(h + 1) * hd], K[kvh], V[kvh], hd, pos + 1, cache_len, hd, scale, False)
            assert np.array_equal(got[h * hd:(h + 1) * hd].view(np.uint32), want.view(np.uint32)), (pos, h)
