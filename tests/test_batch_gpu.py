"""Several sequences decoded together (quintrit_b200_batch_*: one batched pass over the weights per step, attention per sequence over its own KV
cache) against every sequence decoded alone. The reference has one sequence per session and one token per step (quintrit-runtime/src/engine.rs:282,
626-631), so the answer for a batch is what each sequence gives by itself: logits bit for bit, greedy tokens identical."""
import numpy as np
import pytest

import oracle
import quintrit_b200 as q
from quintrit_b200 import synth

pytestmark = pytest.mark.gpu


def _spec(arch, f32_values, config, ctx=1024, hidden=256, **kw):
    return synth.make_model(arch, f32_values, hidden, 512, 2, 4, 2, 64, 300, ctx, 500000.0, 1e-5, config=config, random_norms=True, **kw)


def _alone(spec, tokens, steps):
    """One sequence by itself, token by token: the logits of the prompt's last token and of every generated step, and the generated tokens."""
    d = q.Decoder(spec)
    for pos, t in enumerate(tokens):
        lg, nxt = d.forward(int(t), pos)
    logits, out = [lg], [nxt]
    for k in range(steps):
        lg, nxt = d.forward(out[-1], len(tokens) + k)
        logits.append(lg)
        out.append(nxt)
    d.free()
    return logits, out


@pytest.mark.parametrize("arch,f32_values,hidden", [(q.ARCH_LLAMA, False, 256), (q.ARCH_LLAMA, True, 256), (q.ARCH_BITNET, False, 256), (q.ARCH_LLAMA, False, 288)])
def test_batch_equals_every_sequence_alone(arch, f32_values, hidden):
    spec = _spec(arch, f32_values, 91 + hidden, hidden=hidden, tied=arch == q.ARCH_BITNET)
    lengths = [3, 250, 41, 509, 17]  # two of them cross a 256-position boundary of the padded KV axis while generating
    steps = 9
    prompts = [synth.prompt_tokens(40 + i, n, spec["vocab"]) for i, n in enumerate(lengths)]
    want = [_alone(spec, p, steps) for p in prompts]
    d = q.Decoder(spec)
    b = q.Batch(d, len(prompts))
    for s, p in enumerate(prompts):
        lg, nxt = b.prefill(s, p)
        assert np.array_equal(lg.view(np.uint32), want[s][0][0].view(np.uint32)) and nxt == want[s][1][0], f"prompt of sequence {s}"
    assert list(b.positions()) == lengths
    for k in range(steps):
        toks, lg = b.step(want_logits=True)
        for s in range(len(prompts)):
            assert np.array_equal(lg[s].view(np.uint32), want[s][0][k + 1].view(np.uint32)), f"step {k}, sequence {s}"
            assert toks[s] == want[s][1][k + 1]
    assert list(b.positions()) == [n + steps for n in lengths]
    b.free()
    d.free()


def test_the_oracle_agrees_with_a_batched_step():
    spec = _spec(q.ARCH_LLAMA, False, 95)
    prompts = [synth.prompt_tokens(50 + i, n, spec["vocab"]) for i, n in enumerate([12, 30])]
    d = q.Decoder(spec)
    b = q.Batch(d, 2)
    nxt = [b.prefill(s, p)[1] for s, p in enumerate(prompts)]
    _, lg = b.step(want_logits=True)
    for s, p in enumerate(prompts):
        ref = oracle.Model(spec)
        for pos, t in enumerate(p):
            ref.forward(int(t), pos)
        r = ref.forward(int(nxt[s]), len(p))
        assert np.array_equal(lg[s].view(np.uint32), r.view(np.uint32))


def test_subsets_given_tokens_and_rewind():
    spec = _spec(q.ARCH_LLAMA, False, 96)
    prompts = [synth.prompt_tokens(60 + i, n, spec["vocab"]) for i, n in enumerate([20, 33, 7, 64])]
    want = [_alone(spec, p, 4) for p in prompts]
    d = q.Decoder(spec)
    b = q.Batch(d, 4)
    for s in (2, 0, 3, 1):  # any order
        b.prefill(s, prompts[s][:5])
        b.prefill(s, prompts[s][5:])  # a prompt in two calls
    # sequences 3 and 1 take two steps while 0 and 2 wait; listed in an order of the caller's choosing
    for k in range(2):
        toks, lg = b.step(sequences=[3, 1], want_logits=True)
        assert toks[0] == want[3][1][k + 1] and toks[1] == want[1][1][k + 1]
        assert np.array_equal(lg[0].view(np.uint32), want[3][0][k + 1].view(np.uint32))
    # then all four, the lagging ones catch up; tokens given explicitly are the ones each sequence chose
    given = [want[0][1][0], want[1][1][2], want[2][1][0], want[3][1][2]]
    toks, _ = b.step(tokens=given)
    assert list(toks) == [want[0][1][1], want[1][1][3], want[2][1][1], want[3][1][3]]
    # a slot is rewound and reused for another prompt
    b.rewind(2, 0)
    lg, nxt = b.prefill(2, prompts[3])
    assert np.array_equal(lg.view(np.uint32), want[3][0][0].view(np.uint32)) and nxt == want[3][1][0]
    # the decoder's own cache is untouched by its batches: it still decodes a sequence of its own
    own = [d.forward(int(t), pos) for pos, t in enumerate(prompts[0])][-1]
    assert np.array_equal(own[0].view(np.uint32), want[0][0][0].view(np.uint32))


def test_arguments():
    spec = _spec(q.ARCH_LLAMA, False, 97, ctx=256)
    d = q.Decoder(spec)
    with pytest.raises(q.QuintritError) as e:
        q.Batch(d, 0)
    assert e.value.code == 2
    with pytest.raises(q.QuintritError) as e:
        q.Batch(d, 257)
    assert e.value.code == 2
    b = q.Batch(d, 3)
    with pytest.raises(q.QuintritError) as e:
        b.step()  # nothing to continue from
    assert e.value.code == 2
    with pytest.raises(q.QuintritError) as e:
        b.prefill(3, [1, 2])
    assert e.value.code == 2
    with pytest.raises(q.QuintritError) as e:
        b.prefill(0, np.zeros(300, np.uint32))
    assert e.value.code == 11
    with pytest.raises(q.QuintritError) as e:
        b.prefill(0, [100000])
    assert e.value.code == 2
    b.prefill(0, [1, 2, 3])
    with pytest.raises(q.QuintritError) as e:
        b.step(sequences=[0, 0])
    assert e.value.code == 2 and "twice" in str(e.value)
    with pytest.raises(q.QuintritError) as e:
        b.rewind(0, 9)
    assert e.value.code == 2
    b.prefill(1, np.zeros(256, np.uint32))
    with pytest.raises(q.QuintritError) as e:
        b.step(sequences=[1])
    assert e.value.code == 11  # the context window is full
    toks, _ = b.step(sequences=[0])
    assert toks.shape == (1,) and list(b.positions()) == [4, 256, 0]
    b.free()
    b.free()  # a second free is harmless
    with pytest.raises(q.QuintritError) as e:
        b.step()
    assert e.value.code == 14


def test_block_scaled_decoders_have_no_batch():
    from quintrit_b200 import gguf_io

    spec = synth.make_model(q.ARCH_LLAMA, True, 320, 704, 2, 4, 2, 64, 300, 256, 500000.0, 1e-5, config=98, random_norms=True)
    shapes = [(256, 320), (128, 320), (128, 320), (320, 256), (704, 320), (704, 320), (320, 704)]
    rng = np.random.default_rng(98)
    payloads = []
    for l in range(2):
        for p, (r, c) in enumerate(shapes):
            trits = synth.trits(synth.seed_for(98, l, p, 0), r * c).reshape(r, c)
            payloads.append((q.SRC_Q2_0, gguf_io.encode_q2_0(trits, rng.uniform(0.5, 2.0, r * c // 64).astype(np.float16))))
    d = q.Decoder(dict(spec, weights=payloads))
    with pytest.raises(q.QuintritError) as e:
        q.Batch(d, 2)
    assert e.value.code == 6
