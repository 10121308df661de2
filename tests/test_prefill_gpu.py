"""Prompt ingestion in chunks (quintrit_b200_decoder_prefill: batched projections on the tensor cores, the other steps with a token index in the
grid) against token-by-token decoding: the reference ingests a prompt one token at a time (quintrit-c/src/runtime.rs:430-436), so a batched pass has
to leave the same KV cache, position, logits and greedy choice, bit for bit."""
import numpy as np
import pytest

import oracle
import quintrit_b200 as q
from quintrit_b200 import synth

pytestmark = pytest.mark.gpu


def _spec(arch, f32_values, config, ctx=512, **kw):
    return synth.make_model(arch, f32_values, 256, 512, 2, 4, 2, 64, 300, ctx, 500000.0, 1e-5, config=config, random_norms=True, **kw)


@pytest.mark.parametrize("arch,f32_values,n", [(q.ARCH_LLAMA, False, 40), (q.ARCH_LLAMA, True, 17), (q.ARCH_BITNET, False, 33), (q.ARCH_LLAMA, False, 300)])
def test_chunked_ingestion_equals_single_steps(arch, f32_values, n):
    spec = _spec(arch, f32_values, 21 + n, tied=arch == q.ARCH_BITNET)
    tokens = synth.prompt_tokens(3, n, spec["vocab"])
    a, b = q.Decoder(spec), q.Decoder(spec)
    want = None
    for pos, t in enumerate(tokens):
        want, want_next = a.forward(int(t), pos)
    got, got_next = b.prefill(tokens)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)) and got_next == want_next
    # both continue identically (the cache and the position are the same)
    for step in range(6):
        la, ta = a.forward(want_next, n + step)
        lb, tb = b.forward(got_next, n + step)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)) and ta == tb
        want_next = got_next = ta
    # and the oracle agrees with the last logits
    ref = oracle.Model(spec)
    for pos, t in enumerate(tokens):
        r = ref.forward(int(t), pos)
    assert np.array_equal(got.view(np.uint32), r.view(np.uint32))


@pytest.mark.parametrize("heads,kv_heads,off", [(8, 1, False), (4, 2, True)])
def test_chunks_with_one_query_head_per_attention_block(monkeypatch, heads, kv_heads, off):
    """Where no attention kernel for the whole group of query heads exists (eight heads per KV head) or it is switched off, the
    kernel with one query head per block serves the tokens of a chunk, each at its own position."""
    if off:
        monkeypatch.setenv("QUINTRIT_B200_ATTN_GQA_OFF", "1")
    spec = synth.make_model(q.ARCH_LLAMA, False, 256, 512, 2, heads, kv_heads, 64, 300, 1024, 500000.0, 1e-5, config=41 + heads, random_norms=True)
    tokens = synth.prompt_tokens(7, 600, spec["vocab"])  # past 512 positions: all four KV chunks in use
    a, b = q.Decoder(spec), q.Decoder(spec)
    for pos, t in enumerate(tokens):
        want, want_next = a.forward(int(t), pos, want_logits=pos == len(tokens) - 1)
    got, got_next = b.prefill(tokens)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)) and got_next == want_next


def test_ingestion_in_two_calls_and_after_decoding():
    spec = _spec(q.ARCH_LLAMA, False, 77)
    tokens = synth.prompt_tokens(5, 90, spec["vocab"])
    a, b = q.Decoder(spec), q.Decoder(spec)
    for pos, t in enumerate(tokens):
        want, want_next = a.forward(int(t), pos)
    b.prefill(tokens[:50])
    lg, _ = b.forward(int(tokens[50]), 50)  # a single step in between
    got, got_next = b.prefill(tokens[51:], pos=51)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)) and got_next == want_next
    # rewriting from a shorter prefix (engine_gpu.rs:40-45)
    got2, _ = b.prefill(tokens[10:], pos=10)
    assert np.array_equal(got2.view(np.uint32), want.view(np.uint32))


def test_arguments():
    spec = _spec(q.ARCH_LLAMA, False, 78, ctx=256)
    d = q.Decoder(spec)
    with pytest.raises(q.QuintritError) as e:
        d.prefill(np.zeros(300, np.uint32))
    assert e.value.code == 11
    with pytest.raises(q.QuintritError) as e:
        d.prefill([5], pos=3)  # skips positions
    assert e.value.code == 2
    with pytest.raises(q.QuintritError) as e:
        d.prefill([100000])
    assert e.value.code == 2
    with pytest.raises(q.QuintritError) as e:
        d.prefill([])
    assert e.value.code == 2


def test_many_chunks_replay_one_graph():
    """From the third full chunk on the launches of a chunk are replayed as a CUDA graph: 800 tokens = 3 full chunks + a tail."""
    spec = _spec(q.ARCH_LLAMA, False, 79, ctx=1024)
    tokens = synth.prompt_tokens(6, 800, spec["vocab"])
    a, b = q.Decoder(spec), q.Decoder(spec)
    for pos, t in enumerate(tokens):
        want, want_next = a.forward(int(t), pos)
    got, got_next = b.prefill(tokens)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)) and got_next == want_next
    again, _ = b.prefill(tokens)  # a second prompt on the same decoder: every full chunk is a replay now
    assert np.array_equal(again.view(np.uint32), want.view(np.uint32))
    la, ta = a.forward(want_next, 800)
    lb, tb = b.forward(got_next, 800)
    assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)) and ta == tb
