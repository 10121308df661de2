"""GPU parity of the whole-token decoder through the C ABI against the CPU oracle: logits bit for bit, greedy tokens equal.

Mirrors rust/crates/quintrit-c/tests/engine_gpu.rs:23-100 (a small synthetic model, logits bit-equal at every position,
positions crossing the 256 / 512 padding and the split-KV borders, restart from a shorter prefix) and
rust/crates/quintrit-runtime/tests/gpu_layers.rs:346-408 (head geometries).
"""
import numpy as np
import pytest

import quintrit_b200 as q
from quintrit_b200 import synth

pytestmark = pytest.mark.gpu


def _run(spec, tokens, oracle, check_every=1):
    dec = q.Decoder(spec)
    ref = oracle.Model(spec)
    for pos, tok in enumerate(tokens):
        want = ref.forward(int(tok), pos)
        got, greedy = dec.forward(int(tok), pos, want_logits=(pos % check_every == 0 or pos == len(tokens) - 1))
        if got is not None:
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"logits differ at position {pos}"
        assert greedy == oracle.argmax(want), pos
    return dec, ref


@pytest.mark.parametrize("arch,f32_values,q_heads,kv_heads,head_dim", [
    (q.ARCH_LLAMA, False, 4, 2, 64), (q.ARCH_LLAMA, True, 4, 2, 64), (q.ARCH_BITNET, False, 4, 1, 128),
    (q.ARCH_BITNET, True, 2, 2, 128), (q.ARCH_LLAMA, False, 3, 1, 256), (q.ARCH_LLAMA, False, 4, 4, 32)])
def test_logits_are_bit_equal_at_every_position(oracle, arch, f32_values, q_heads, kv_heads, head_dim):
    hidden = 320 if head_dim != 256 else 512
    spec = synth.make_model(arch, f32_values, hidden, 704, 2, q_heads, kv_heads, head_dim, 300, 256, 500000.0, 1e-5, config=9, random_norms=True)
    rng = np.random.default_rng(1)
    _run(spec, rng.integers(0, 300, 40), oracle)


@pytest.mark.parametrize("f32_values", [False, True])
def test_long_context_crosses_every_split_border(oracle, f32_values):
    # context 1280 as the reference's engine test: 255 / 256 / 257, 511 / 512 / 513, chunk borders of 768, 1024, 1280
    spec = synth.make_model(q.ARCH_LLAMA, f32_values, 128, 256, 1, 2, 1, 64, 264, 1280, 10000.0, 1e-6, config=11, tied=True)
    rng = np.random.default_rng(2)
    _run(spec, rng.integers(0, 264, 1100), oracle, check_every=1)


def test_restart_from_a_shorter_prefix_and_generate(oracle):
    spec = synth.make_model(q.ARCH_BITNET, False, 256, 512, 2, 4, 2, 64, 500, 512, 500000.0, 1e-5, config=12, tied=True)
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, 500, 24)
    dec, ref = _run(spec, prompt, oracle)
    # rewrite positions 10.. with other tokens (engine_gpu.rs:40-45)
    other = rng.integers(0, 500, 8)
    for i, tok in enumerate(other):
        want = ref.forward(int(tok), 10 + i)
        got, _ = dec.forward(int(tok), 10 + i)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # greedy generation on the device equals the oracle's loop
    ref2 = oracle.Model(spec)
    tok = None
    for pos, t in enumerate(prompt):
        tok = oracle.argmax(ref2.forward(int(t), pos))
    want_tokens = [tok]
    for j in range(1, 48):
        tok = oracle.argmax(ref2.forward(int(tok), len(prompt) + j - 1))
        want_tokens.append(tok)
    got_tokens = dec.generate(prompt, 48)
    assert list(got_tokens) == want_tokens
    assert dec.time_token(2, 5) > 0


def test_invalid_decoder_calls():
    spec = synth.make_model(q.ARCH_LLAMA, False, 128, 256, 1, 2, 1, 64, 64, 256, 10000.0, 1e-5, config=13, tied=True)
    dec = q.Decoder(spec)
    with pytest.raises(q.QuintritError) as e:
        dec.forward(64, 0)
    assert e.value.code == 2
    with pytest.raises(q.QuintritError) as e:
        dec.forward(1, 3)  # skips positions
    assert e.value.code == 2
    with pytest.raises(q.QuintritError) as e:
        dec.generate(np.arange(10), 300)
    assert e.value.code == 11
    bad = dict(spec, head_dim=48, q_heads=2, kv_heads=1)
    with pytest.raises(q.QuintritError):
        q.Decoder(bad)


@pytest.mark.parametrize("arch", [q.ARCH_LLAMA, q.ARCH_BITNET])
def test_bf16_embedding_and_head(oracle, arch):
    """BF16 tables with the reference's BF16 projection arithmetic (hybrid.rs:327-333, ops.rs:650-712): the single-kernel path
    (LLaMA) and the one-kernel-per-step path (BitNet) against the oracle."""
    spec = synth.make_model(arch, False, 320, 704, 2, 4, 2, 64, 300, 256, 500000.0, 1e-5, config=17, random_norms=True, bf16_tables=True,
                            tied=(arch == q.ARCH_BITNET))
    dec, _ = _run(spec, synth.prompt_tokens(6, 10, spec["vocab"]), oracle)
    assert dec.info()["table_dtype"] == 1
    dec.free()


def _q2_0_model(arch, config):
    """A model whose projections are Q2_0 blocks (f16 scale per 64 weights): the device gets the GGUF payloads, the oracle the
    planar bytes and the widened scales."""
    from quintrit_b200 import gguf_io

    spec = synth.make_model(arch, True, 320, 704, 2, 4, 2, 64, 300, 256, 500000.0, 1e-5, config=config, random_norms=True, tied=(arch == q.ARCH_BITNET))
    shapes = [(256, 320), (128, 320), (128, 320), (320, 256), (704, 320), (704, 320), (320, 704)]
    rng = np.random.default_rng(config)
    payloads, block_scales = [], []
    for l in range(2):
        for p, (r, c) in enumerate(shapes):
            trits = synth.trits(synth.seed_for(config, l, p, 0), r * c).reshape(r, c)
            sc = rng.uniform(0.5, 2.0, r * c // 64).astype(np.float16)
            payloads.append((q.SRC_Q2_0, gguf_io.encode_q2_0(trits, sc)))
            block_scales.append(sc.astype(np.float32))
    return dict(spec, block_scales=block_scales), payloads


@pytest.mark.parametrize("arch", [q.ARCH_LLAMA, q.ARCH_BITNET])
def test_q2_0_model_decodes_like_the_oracle(oracle, arch):
    """Block-scaled projections in the whole decoder (attention.rs:262-344, model.rs:209-229): Q8_0 activation blocks, F32
    projection results, FP32-accumulator attention."""
    spec, payloads = _q2_0_model(arch, 23)
    dec = q.Decoder(dict(spec, weights=payloads))
    assert dec.info()["single_kernel"] == 0
    ref = oracle.Model(spec)
    for pos, tok in enumerate(synth.prompt_tokens(9, 14, spec["vocab"])):
        want = ref.forward(int(tok), pos)
        got, greedy = dec.forward(int(tok), pos)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"logits differ at position {pos}"
        assert greedy == oracle.argmax(want)
    dec.free()
    # a model may not mix block-scaled and per-tensor projections
    mixed = list(payloads)
    mixed[3] = spec["weights"][3]
    with pytest.raises(q.QuintritError) as e:
        q.Decoder(dict(spec, weights=mixed))
    assert e.value.code == 6


def _head_norms(spec, seed):
    rng = np.random.default_rng(seed)
    return [rng.uniform(0.5, 1.5, spec["head_dim"]).astype(np.float32) for _ in range(spec["layers"] * 2)]


def test_qwen3_shape_with_query_and_key_head_norms(oracle):
    """Qwen3: every query and key head is RMS-normalised with its own weights before NEOX RoPE (attention.rs:282-294,
    config.rs:424, 464-467); only block-scaled models have it, as in the reference."""
    spec, payloads = _q2_0_model(q.ARCH_LLAMA, 29)
    spec = dict(spec, arch=q.ARCH_QWEN, qk_norms=_head_norms(spec, 5))
    dec = q.Decoder(dict(spec, weights=payloads))
    ref, plain = oracle.Model(spec), oracle.Model({k: v for k, v in spec.items() if k != "qk_norms"})
    for pos, tok in enumerate(synth.prompt_tokens(6, 12, spec["vocab"])):
        want = ref.forward(int(tok), pos)
        got, greedy = dec.forward(int(tok), pos)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"logits differ at position {pos}"
        assert greedy == oracle.argmax(want)
        other = plain.forward(int(tok), pos)
        assert pos == 0 or not np.array_equal(want, other)  # the head norms change the result once there is more than one key
    dec.free()
    per_tensor = synth.make_model(q.ARCH_QWEN, True, 320, 704, 2, 4, 2, 64, 300, 256, 500000.0, 1e-5, config=29)
    with pytest.raises(q.QuintritError) as e:
        q.Decoder(dict(per_tensor, qk_norms=_head_norms(per_tensor, 5)))
    assert e.value.code == 6


@pytest.mark.parametrize("f32_values", [False, True])
def test_qwen2_shape_rotates_neox_pairs_and_keeps_swiglu(oracle, f32_values):
    """Qwen2: LLaMA blocks with NEOX RoPE pairs (config.rs:464-467), on the single-kernel path and in prompt chunks."""
    spec = synth.make_model(q.ARCH_QWEN, f32_values, 320, 704, 2, 4, 2, 64, 300, 256, 500000.0, 1e-5, config=31, random_norms=True)
    toks = synth.prompt_tokens(8, 20, spec["vocab"])
    dec, _ = _run(spec, toks[:10], oracle)
    ref = oracle.Model(spec)
    for pos, tok in enumerate(toks):
        want = ref.forward(int(tok), pos)
    got, _ = dec.prefill(toks, 0)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    llama = oracle.Model(dict(spec, arch=q.ARCH_LLAMA))
    for pos, tok in enumerate(toks):
        other = llama.forward(int(tok), pos)
    assert not np.array_equal(other, want)
    dec.free()


@pytest.mark.parametrize("arch,f32_values", [(q.ARCH_LLAMA, False), (q.ARCH_BITNET, True)])
def test_one_kernel_per_step_path_stays_exact(oracle, monkeypatch, arch, f32_values):
    """Both decode paths serve both architectures; QUINTRIT_B200_DECODE=kernels selects the one-kernel-per-step path, which
    otherwise only runs for shapes the token kernel does not take."""
    monkeypatch.setenv("QUINTRIT_B200_DECODE", "kernels")
    spec = synth.make_model(arch, f32_values, 320, 704, 2, 4, 2, 64, 300, 256, 500000.0, 1e-5, config=19, random_norms=True, tied=(arch == q.ARCH_BITNET))
    dec, _ = _run(spec, synth.prompt_tokens(4, 10, spec["vocab"]), oracle)
    assert dec.info()["single_kernel"] == 0
    dec.free()
    monkeypatch.delenv("QUINTRIT_B200_DECODE")
    dec2 = q.Decoder(spec)
    assert dec2.info()["single_kernel"] == 1
    dec2.free()


@pytest.mark.parametrize("f32_values,head_dim,q_heads,kv_heads", [(False, 256, 3, 1), (True, 128, 4, 2)])
def test_context_of_several_thousand_positions(oracle, f32_values, head_dim, q_heads, kv_heads):
    """Chunks of more than a thousand positions: the staged key blocks take several rounds per CTA, the V slice of a chunk no
    longer fits one copy group comfortably, the next-moved table spans more than 32 groups. Context 3584 (the reference caps
    its GPU sessions at 7936, gpu.rs:141-146); logits are compared at a sample of positions and at the last one."""
    hidden = q_heads * head_dim // 2 if head_dim == 256 else 256
    spec = synth.make_model(q.ARCH_LLAMA, f32_values, hidden, 256, 1, q_heads, kv_heads, head_dim, 264, 3584, 10000.0, 1e-6, config=29, tied=True)
    rng = np.random.default_rng(5)
    _run(spec, rng.integers(0, 264, 3400), oracle, check_every=211)
