"""Models loaded from synthetic GGUF files through quintrit_b200_decoder_open_gguf against the CPU oracle built from the
same tensors: logits bit for bit and identical greedy tokens for each ternary encoding (I2_S -> FP16-accumulator
attention, TQ1_0 / TQ2_0 -> FP32 accumulators, as rust/crates/quintrit-runtime/src/config.rs:425-429 selects), a BitNet
file with sub-norms and a tied head, and the loader's rejections (rust/crates/quintrit-runtime/src/gpu.rs:149-181)."""
import struct

import numpy as np
import pytest

import oracle
import quintrit_b200 as q
from quintrit_b200 import gguf_io, synth

pytestmark = pytest.mark.gpu


def _model(arch, f32_values, config, tied=False):
    spec = synth.make_model(arch, f32_values, 256, 512, 2, 4, 2, 64, 300, 512, 500000.0, 1e-5, config=config, random_norms=True, tied=tied)
    shapes = [(256, 256), (128, 256), (128, 256), (256, 256), (512, 256), (512, 256), (256, 512)]
    trits = [synth.trits(synth.seed_for(config, l, p, 0), r * c).reshape(r, c) for l in range(2) for p, (r, c) in enumerate(shapes)]
    return spec, trits


@pytest.mark.parametrize("encoding,f32_values", [(gguf_io.GGML_I2_S, False), (gguf_io.GGML_TQ2_0, True), (gguf_io.GGML_TQ1_0, True)])
def test_llama_file_decodes_like_the_oracle(tmp_path, encoding, f32_values):
    spec, trits = _model(q.ARCH_LLAMA, f32_values, 11)
    if encoding != gguf_io.GGML_I2_S:
        spec["scales"] = np.float32(np.float16(spec["scales"]))  # the tensor scale is the f16 of every block
    path = tmp_path / "model.gguf"
    gguf_io.write_model_gguf(path, spec, trits, encoding)
    dec = q.Decoder.open(path)
    info = dec.info()
    assert (info["hidden_size"], info["num_layers"], info["num_heads"], info["num_kv_heads"], info["head_dim"], info["vocab_size"]) == (256, 2, 4, 2, 64, 300)
    assert info["f32_values"] == int(f32_values) and info["context_length"] == 512 and info["arch"] == q.ARCH_LLAMA
    ref = oracle.Model(spec)
    tokens = synth.prompt_tokens(3, 12, spec["vocab"])
    for pos, tok in enumerate(tokens):
        want = ref.forward(int(tok), pos)
        got, greedy = dec.forward(int(tok), pos)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (encoding, pos)
        assert greedy == oracle.argmax(want)
    # generate from the file-backed decoder = greedy loop of the oracle
    out = dec.generate(tokens[:4], 5)
    ref2 = oracle.Model(spec)
    for pos, tok in enumerate(tokens[:4]):
        last = ref2.forward(int(tok), pos)
    want_tokens = []
    for i in range(5):
        t = oracle.argmax(last)
        want_tokens.append(t)
        last = ref2.forward(t, 4 + i)
    assert list(out) == want_tokens
    dec.free()


def test_bitnet_file_with_sub_norms_and_tied_head(tmp_path):
    spec, trits = _model(q.ARCH_BITNET, False, 12, tied=True)
    path = tmp_path / "bitnet.gguf"
    gguf_io.write_model_gguf(path, spec, trits, gguf_io.GGML_I2_S, architecture="bitnet-b1.58")
    dec = q.Decoder.open(path, context=256)
    assert dec.info()["arch"] == q.ARCH_BITNET and dec.info()["context_length"] == 256
    spec = dict(spec, ctx=256)
    ref = oracle.Model(spec)
    for pos, tok in enumerate(synth.prompt_tokens(4, 6, spec["vocab"])):
        want = ref.forward(int(tok), pos)
        got, _ = dec.forward(int(tok), pos)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), pos
    dec.free()


def test_rejections(tmp_path):
    spec, trits = _model(q.ARCH_LLAMA, False, 13)

    def code(path, **kw):
        with pytest.raises(q.QuintritError) as e:
            q.Decoder.open(path, **kw)
        return e.value.code, str(e.value)

    assert code(tmp_path / "nope.gguf")[0] == 7
    junk = tmp_path / "junk.gguf"
    junk.write_bytes(b"not a model" * 10)
    assert code(junk)[0] == 8
    good = tmp_path / "good.gguf"
    gguf_io.write_model_gguf(good, spec, trits, gguf_io.GGML_I2_S)
    assert code(good, flags=2)[0] == 2                      # unknown flag bits (1 = QUINTRIT_MODEL_OPEN_VERBOSE is accepted and changes nothing)
    assert code(good, context=100)[0] == 2                  # a window below 256 positions is kept as it is (gpu.rs:141-146) but must be a multiple of 8
    small = q.Decoder.open(good, context=96, flags=1)
    assert small.info()["context_length"] == 96
    small.free()
    meta = {"general.architecture": "llama", "llama.embedding_length": 256, "llama.attention.head_count": 4, "llama.vocab_size": 300}
    # a missing projection names the tensor
    miss = tmp_path / "miss.gguf"
    gguf_io.write_gguf(miss, dict(meta, **{"llama.block_count": 1, "llama.feed_forward_length": 512, "llama.attention.head_count_kv": 2,
                                          "llama.attention.key_length": 64, "llama.context_length": 512}), [])
    c, msg = code(miss)
    assert c == 10 and "blk.0.attn_q.weight" in msg
    # payloads cut off: format error, not a crash
    raw = good.read_bytes()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(raw[: len(raw) // 2])
    assert code(cut)[0] in (8, 10)
    # TQ tensor whose blocks disagree on the scale is not a ternary projection (decoders/mod.rs:121-138)
    spec2 = dict(spec, scales=np.float32(np.float16(spec["scales"])))
    tq = tmp_path / "tq.gguf"
    gguf_io.write_model_gguf(tq, spec2, trits, gguf_io.GGML_TQ2_0)
    data = bytearray(tq.read_bytes())
    d = q.gguf_describe(tq)
    first = next(t for t in d["tensors"] if t["name"] == "blk.0.attn_q.weight")
    # find the payload: the second block's scale bytes sit 66 + 64 bytes into it; locate it through the known first block
    blk = gguf_io.encode_tq2_0(trits[0], int(np.float16(spec2["scales"][0]).view(np.uint16))).tobytes()
    at = bytes(data).find(blk[:132])
    assert at > 0 and first["bytes"] == len(blk)
    data[at + 66 + 64] ^= 0x01
    tq.write_bytes(bytes(data))
    c, msg = code(tq)
    assert c == 6 and "block scales" in msg


def test_bf16_tables_from_a_file(tmp_path):
    spec = synth.make_model(q.ARCH_LLAMA, False, 256, 512, 2, 4, 2, 64, 300, 512, 500000.0, 1e-5, config=14, random_norms=True, bf16_tables=True)
    shapes = [(256, 256), (128, 256), (128, 256), (256, 256), (512, 256), (512, 256), (256, 512)]
    trits = [synth.trits(synth.seed_for(14, l, p, 0), r * c).reshape(r, c) for l in range(2) for p, (r, c) in enumerate(shapes)]
    path = tmp_path / "bf16.gguf"
    gguf_io.write_model_gguf(path, spec, trits, gguf_io.GGML_I2_S)
    assert any(t["name"] == "output.weight" and t["type"] == 30 for t in q.gguf_describe(path)["tensors"])
    dec = q.Decoder.open(path)
    assert dec.info()["table_dtype"] == 1
    ref = oracle.Model(spec)
    for pos, tok in enumerate(synth.prompt_tokens(8, 6, spec["vocab"])):
        want = ref.forward(int(tok), pos)
        got, _ = dec.forward(int(tok), pos)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), pos
    dec.free()


def test_q2_0_file(tmp_path):
    """A whole model of Q2_0 projections from a file (the reference's GPU loader refuses these, gpu.rs:152-154; its CPU path is
    the oracle's): logits bit for bit."""
    spec = synth.make_model(q.ARCH_LLAMA, True, 256, 512, 2, 4, 2, 64, 300, 512, 500000.0, 1e-5, config=15, random_norms=True)
    shapes = [(256, 256), (128, 256), (128, 256), (256, 256), (512, 256), (512, 256), (256, 512)]
    trits = [synth.trits(synth.seed_for(15, l, p, 0), r * c).reshape(r, c) for l in range(2) for p, (r, c) in enumerate(shapes)]
    rng = np.random.default_rng(15)
    spec["block_scales"] = [rng.uniform(0.5, 2.0, t.size // 64).astype(np.float16).astype(np.float32) for t in trits]
    path = tmp_path / "q2.gguf"
    gguf_io.write_model_gguf(path, spec, trits, gguf_io.GGML_Q2_0)
    dec = q.Decoder.open(path)
    assert dec.info()["f32_values"] == 1 and dec.info()["single_kernel"] == 0
    ref = oracle.Model(spec)
    for pos, tok in enumerate(synth.prompt_tokens(8, 8, spec["vocab"])):
        want = ref.forward(int(tok), pos)
        got, _ = dec.forward(int(tok), pos)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), pos
    dec.free()
