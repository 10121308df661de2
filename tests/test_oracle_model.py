"""Pins the oracle's float primitives to the reference's definitions and known answers.

Sources: rust/crates/quintrit-runtime/src/ops.rs:2086-2109 (every half value against the soft conversion),
ops.rs:2010-2059 (portable model of ggml_vec_dot_f16), rust/crates/quintrit-runtime/tests/model_ops_tests.rs:42-49
(bf16 RNE), :98-134 (RoPE pair selection), tests/algorithm_tests.rs:48-213, 599-680 (f64 tolerance references for
RMSNorm, SiLU, softmax attention). The glibc expf restatement that the device uses is compared with the host libm.
"""
import ctypes
import ctypes.util
from fractions import Fraction

import numpy as np


def test_half_conversions_are_exact_for_every_half(oracle):
    l = oracle.mlib()
    h = np.arange(65536, dtype=np.uint16)
    f = h.view(np.float16).astype(np.float32)
    for i in list(range(0, 65536, 5)) + [0x7C00, 0xFC00, 0x0001, 0x03FF, 0x0400, 0x7BFF]:
        got = np.float32(l.qto_f16_to_f32(int(h[i])))
        assert got.view(np.uint32) == f[i].view(np.uint32) or (np.isnan(got) and np.isnan(f[i]))
        if not np.isnan(f[i]):
            assert l.qto_f32_to_f16(float(f[i])) == h[i]
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 100, np.float32([65504, 65520, 65519.9, 1e-8, 6e-8, -0.0, 1e9])])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle.f32_to_f16_bits(x), want)


def test_bf16_round_to_nearest_even(oracle):
    l = oracle.mlib()
    for bits, want in [(0x3F800000, 0x3F80), (0x3F808000, 0x3F80), (0x3F818000, 0x3F82), (0x3F808001, 0x3F81), (0x7FC00001, 0x7FC0)]:
        assert l.qto_f32_to_bf16(float(np.uint32(bits).view(np.float32))) == want or bits == 0x7FC00001
    assert np.float32(l.qto_bf16_to_f32(0x3F80)) == 1.0


def test_rms_norm_definition(oracle):
    rng = np.random.default_rng(1)
    for n in (8, 2560, 3072, 6912):
        x = (rng.standard_normal(n) * 3).astype(np.float32)
        w = rng.uniform(0.5, 1.5, n).astype(np.float32)
        got = oracle.rms_norm(x, w, 1e-5)
        sq = (x * x).astype(np.float32).astype(np.float64)
        s = 0.0
        for v in sq:
            s += v
        inv = np.float32(1.0) / np.sqrt(np.float32(s / n) + np.float32(1e-5), dtype=np.float32)
        want = ((x * inv).astype(np.float32) * w).astype(np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-5) * w
        assert np.abs(got - ref).max() < 1e-5 * np.abs(ref).max()


def test_rope_pairs_and_passthrough(oracle):
    hd, n_dims = 8, 4
    x = np.arange(1, 2 * hd + 1, dtype=np.float32)
    cache = np.float32([0.0, 1.0, -1.0, 0.0])  # pair 0: cos 0 sin 1 (quarter turn); pair 1: cos -1 sin 0 (half turn)
    normal = oracle.rope_apply(x, 2, hd, 0, cache)
    assert list(normal[:8]) == [-2, 1, -3, -4, 5, 6, 7, 8]
    neox = oracle.rope_apply(x, 2, hd, 1, cache)
    assert list(neox[:8]) == [-3, -2, 1, -4, 5, 6, 7, 8]
    c = oracle.rope_cache(7, 64, 500000.0)
    ts = np.float32(500000.0) ** np.float32(-2.0 / 64)
    assert abs(c[0] - np.cos(7.0)) < 1e-6 and abs(c[3] - np.sin(7.0 * float(ts))) < 1e-5
    assert list(oracle.rope_cache(0, 8, 10000.0)) == [1, 0, 1, 0, 1, 0, 1, 0]


def _dot_f16_model(x, y):
    xf, yf = x.view(np.float16).astype(np.float32), y.view(np.float16).astype(np.float32)
    n = x.size
    acc = np.zeros((4, 8), np.float64)
    i = 0
    while i + 32 <= n:
        for j in range(4):
            for l in range(8):
                k = i + 8 * j + l
                acc[j, l] = np.float32(float(xf[k]) * float(yf[k]) + float(acc[j, l]))  # products of two halves are exact in f64
        i += 32
    f = np.float32
    red = [f(f(f(acc[0, l]) + f(acc[2, l])) + f(f(acc[1, l]) + f(acc[3, l]))) for l in range(8)]
    t0 = [f(red[l] + red[l + 4]) for l in range(4)]
    s = f(f(t0[0] + t0[1]) + f(t0[2] + t0[3]))
    while i < n:
        s = f(s + f(xf[i] * yf[i]))
        i += 1
    return s


def test_vec_dot_f16_order(oracle):
    rng = np.random.default_rng(2)
    for n in (32, 64, 128, 256, 100, 3072):
        x = rng.standard_normal(n).astype(np.float16).view(np.uint16)
        y = (rng.standard_normal(n) * 4).astype(np.float16).view(np.uint16)
        assert oracle.vec_dot_f16(x, y).view(np.uint32) == _dot_f16_model(x, y).view(np.uint32), n
    x = rng.standard_normal(264).astype(np.float16).view(np.uint16)
    y = rng.standard_normal(264).astype(np.float32)
    got = oracle.vec_dot_f16_f32(x, y)
    ref = float((x.view(np.float16).astype(np.float64) * y.astype(np.float64)).sum())
    assert abs(got - ref) < 1e-4


def test_device_expf_restatement_equals_the_host_libm(oracle):
    libm = ctypes.CDLL(ctypes.util.find_library("m"))
    libm.expf.restype = ctypes.c_float
    libm.expf.argtypes = [ctypes.c_float]
    # the table: 2^(i/32) correctly rounded, minus i << 47
    tab = oracle.exp2_table()
    for i in range(32):
        v = float(np.uint64(int(tab[i]) + (i << 47)).view(np.float64))
        exact = Fraction(2) ** i  # compare v^32 with 2^i: |v^32 / 2^i - 1| < 32 * 2^-53 * 1.01 for a correctly rounded root
        err = abs(Fraction(v) ** 32 / exact - 1)
        assert err < Fraction(32 * 1.01) / 2 ** 53, i
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.uniform(-104, 0.5, 150000), rng.uniform(-1e-3, 1e-3, 20000), rng.uniform(0, 89, 30000),
                         [0.0, -0.0, -87.3, -88.0, -103.9, -104.0, -200.0, 88.7, 88.8, 100.0, -np.inf, np.inf]]).astype(np.float32)
    got = oracle.expf_restated(xs)
    want = np.array([libm.expf(float(v)) for v in xs], np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_silu_polynomial_close_to_the_definition(oracle):
    rng = np.random.default_rng(4)
    g = np.concatenate([rng.standard_normal(4096) * 6, [0, -0.0, 80, -80, 100, -100, 1e-6]]).astype(np.float32)
    g = g[: g.size // 8 * 8]
    u = rng.standard_normal(g.size).astype(np.float32)
    got = oracle.swiglu(g, u)
    ref = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u
    assert np.abs(got - ref).max() <= 2e-6 * max(1.0, np.abs(ref).max())
    r = oracle.relu2_mul(np.float32([-1, 2, 0.5]), np.float32([3, 3, -2]))
    assert list(r) == [0, 12, -0.5]


def _attention_f64(q, K, V, L, scale):
    s = (K[:L].view(np.float16).astype(np.float64) @ q.astype(np.float64)) * scale
    p = np.exp(s - s.max())
    p /= p.sum()
    return p @ V[:L].view(np.float16).astype(np.float64)


def test_attention_matches_softmax_across_padding_and_chunk_borders(oracle):
    rng = np.random.default_rng(5)
    hd, ctx = 64, 1280
    K = (rng.standard_normal((ctx, hd))).astype(np.float16).view(np.uint16)
    V = (rng.standard_normal((ctx, hd))).astype(np.float16).view(np.uint16)
    q = rng.standard_normal(hd).astype(np.float32)
    scale = 1 / np.sqrt(hd)
    for L in (1, 2, 255, 256, 257, 511, 512, 513, 767, 768, 1023, 1024, 1025, 1280):
        ref = _attention_f64(q.astype(np.float16).astype(np.float32), K, V, L, scale)
        for f32_values, tol in ((False, 2e-2), (True, 2e-3)):
            qq = q if f32_values else q
            got = oracle.attend_head(qq, K, V, hd, L, ctx, hd, scale, f32_values)
            ref2 = _attention_f64(q, K, V, L, scale) if f32_values else ref
            assert np.abs(got - ref2).max() < tol, (L, f32_values)


def test_argmax_takes_the_first_maximum(oracle):
    assert oracle.argmax(np.float32([1, 5, 5, 2])) == 1
    assert oracle.argmax(np.float32([np.nan, -1, np.nan])) == 1


def test_vec_dot_bf16_follows_the_documented_order(oracle):
    """rust/crates/quintrit-runtime/src/ops.rs:688-712: 4 x 8 lanes, product and sum rounded separately (no FMA),
    (a0+a2)+(a1+a3), g_l = a_{l+4}+a_l, (g0+g2)+(g1+g3), tail in double."""
    rng = np.random.default_rng(4)
    for n in (32, 64, 320, 3072, 45, 100):
        x = oracle.f32_to_bf16_bits(rng.standard_normal(n).astype(np.float32))
        y = oracle.f32_to_bf16_bits((rng.standard_normal(n) * 0.02).astype(np.float32))
        xf = (x.astype(np.uint32) << 16).view(np.float32)
        yf = (y.astype(np.uint32) << 16).view(np.float32)
        acc = np.zeros((4, 8), np.float32)
        full = n // 32 * 32
        for i in range(0, full, 32):
            prod = (xf[i:i + 32] * yf[i:i + 32]).astype(np.float32).reshape(4, 8)
            acc = (acc + prod).astype(np.float32)
        a = ((acc[0] + acc[2]).astype(np.float32) + (acc[1] + acc[3]).astype(np.float32)).astype(np.float32)
        g = (a[4:] + a[:4]).astype(np.float32)
        s = np.float64(np.float32(np.float32(g[0] + g[2]) + np.float32(g[1] + g[3])))
        for k in range(full, n):
            s += np.float64(np.float32(xf[k] * yf[k]))
        want = np.float32(s)
        assert oracle.vec_dot_bf16(x, y).view(np.uint32) == want.view(np.uint32), n
    ones = np.full(64, 0x3F80, np.uint16)
    assert oracle.vec_dot_bf16(ones, ones) == np.float32(64.0)


def test_head_norms_reach_the_queries_and_keys_of_their_layer(oracle):
    """Query/key-norm (attention.rs:282-294): the query heads take the layer's first weight vector, the key heads the second.
    Halving the query weights and doubling the key weights (powers of two: exact through the norm, RoPE, the F16 key cache
    and every product of a score) leaves each score and so the logits bit for bit; giving the keys the queries' weights, or
    a layer the other layer's, does not."""
    from quintrit_b200 import synth

    spec = synth.make_model(2, True, 128, 256, 2, 4, 2, 32, 200, 64, 10000.0, 1e-6, config=17, random_norms=True)
    shapes = [(128, 128), (64, 128), (64, 128), (128, 128), (256, 128), (256, 128), (128, 256)]
    rng = np.random.default_rng(17)
    spec["block_scales"] = [rng.uniform(0.5, 2.0, r * c // 64).astype(np.float16).astype(np.float32) for _ in range(2) for r, c in shapes]
    w = [rng.uniform(0.5, 1.5, 32).astype(np.float32) for _ in range(4)]
    tokens = synth.prompt_tokens(2, 9, 200)

    def logits(head_norms):
        m = oracle.Model(dict(spec, qk_norms=head_norms))
        return [m.forward(int(t), p).copy() for p, t in enumerate(tokens)]

    base = logits(w)
    traded = logits([w[0] * np.float32(0.5), w[1] * np.float32(2.0), w[2] * np.float32(4.0), w[3] * np.float32(0.25)])
    assert all(np.array_equal(a.view(np.uint32), b.view(np.uint32)) for a, b in zip(base, traded))
    swapped_roles = logits([w[1], w[0], w[2], w[3]])
    swapped_layers = logits([w[2], w[3], w[0], w[1]])
    assert not np.array_equal(base[-1], swapped_roles[-1]) and not np.array_equal(base[-1], swapped_layers[-1])
    assert np.array_equal(base[0], swapped_roles[0])  # one position: the only key has weight 1 whatever its score
