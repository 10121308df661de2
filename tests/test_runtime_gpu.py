"""The runtime level of the reference's C API on a B200 (quintrit_model_open_gpu ... quintrit_session_generate, as exported by
libquintrit_b200.so) against the CPU oracle, on the reference's own tiny test model (tests/golden/ref_tiny_model.gguf, written by
the reference's gguf_builder.py). The reference's GPU test asks for bit-identical logits and identical greedy, sampled, streamed
and chat text between its CPU and GPU builds (rust/crates/quintrit-py/tests/test_cuda.py:52-77); the CPU side here is the oracle."""
import ctypes as C
import os
import subprocess
import threading

import numpy as np
import pytest

import oracle
from oracle import gguf_model, sampler
from quintrit_b200 import gguf_io, synth
from quintrit_b200.api import QuintritError
from quintrit_b200.runtime import GgufFile, Model, Tokenizer, _SessionInfo

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = os.path.join(ROOT, "tests", "golden", "ref_tiny_model.gguf")
PROMPT = "the cat sat on the mat"


@pytest.fixture(scope="module")
def gpu():
    m = Model.load(TINY, device="cuda")
    yield m
    m.close()


@pytest.fixture(scope="module")
def cpu():
    return oracle.Model(gguf_model.model_spec(TINY))


@pytest.fixture(scope="module")
def tok():
    return Tokenizer(TINY)


def _oracle_text(cpu, tok, prompt, n, **kw):
    ids = tok.encode(prompt, add_bos=True)
    out, reason = sampler.generate(cpu, ids, n, sampler.Sampler(**kw) if kw else None, eos=tok.eos_token_id)
    return "".join(tok.decode_pieces(out)), out, reason


def test_properties_of_the_model(gpu):
    assert gpu.device == "cuda:0" and gpu.kernel == "cuda" and gpu.threads == 0
    assert gpu.architecture == "llama" and gpu.vocab_size == 261 and gpu.context_length == 64 and gpu.context_window == 64
    assert gpu.n_layers == 2 and gpu.hidden_size == 128
    cfg = gpu.config
    assert (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]) == (4, 2, 32)
    assert cfg["bos_token_id"] == 259 and cfg["eos_token_id"] == 260
    assert "device=" in repr(gpu)


def test_logits_are_bit_identical_to_the_cpu_oracle(gpu, cpu, tok):
    ids = tok.encode(PROMPT, add_bos=True)
    want = None
    for p, t in enumerate(ids):
        want = cpu.forward(t, p)
    got = gpu.logits(ids)
    assert got.dtype == np.float32 and got.shape == (261,)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(gpu.logits(PROMPT).view(np.uint32), want.view(np.uint32))  # text: BOS is put in front
    assert np.array_equal(gpu.logits(ids).view(np.uint32), want.view(np.uint32))  # a repeated call restarts from an empty cache
    # feeding in two parts with KEEP_CONTEXT is the same as feeding at once
    gpu.logits(ids[:7])
    assert np.array_equal(gpu.logits(ids[7:], keep_context=True).view(np.uint32), want.view(np.uint32))
    assert gpu.position == len(ids)
    assert not np.array_equal(gpu.logits("a different prompt"), want)


def test_greedy_sampled_streamed_and_chat_text_match_the_oracle(gpu, cpu, tok):
    want, ids, _ = _oracle_text(cpu, tok, PROMPT, 20)
    assert gpu.generate(PROMPT, 20) == want
    assert gpu.generate(PROMPT, 20, temperature=0.0, top_k=40, top_p=0.9) == want  # temperature 0 is greedy whatever the rest says
    assert np.array_equal(gpu.generate_tokens(tok.encode(PROMPT, add_bos=True), 20), ids)  # the loop that stays on the device
    for seed in (3, 42):
        want_s, _, _ = _oracle_text(cpu, tok, PROMPT, 20, temperature=0.8, top_k=40, top_p=0.9, seed=seed)
        assert gpu.generate(PROMPT, 20, temperature=0.8, seed=seed) == want_s
    want_k0, _, _ = _oracle_text(cpu, tok, PROMPT, 12, temperature=1.3, top_k=0, top_p=1.0, seed=7)  # neither top-k nor nucleus: no sorting at all
    assert gpu.generate(PROMPT, 12, temperature=1.3, top_k=0, top_p=1.0, seed=7) == want_k0
    s = gpu.stream(PROMPT, 12)
    assert s.text == s.buffer_text == gpu.generate(PROMPT, 12) and s.n_tokens <= 12 and s.finish_reason in ("length", "eos")
    assert "".join(s) == s.text and list(s) == []
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    prompt = gpu.format_chat(msgs)
    assert prompt == "### System:\nbe brief\n\n### User:\nhi\n\n### Assistant:\n"  # engine.rs:95-118, a model that is not Falcon3
    assert gpu.chat(msgs, 6) == gpu.generate(prompt, 6) == _oracle_text(cpu, tok, prompt, 6)[0]


def test_lengths_stops_context_and_errors(gpu, cpu, tok):
    assert gpu.generate(PROMPT, 0) == ""
    short, longer = gpu.generate(PROMPT, 4), gpu.generate(PROMPT, 9)
    assert longer.startswith(short)
    free = gpu.generate(PROMPT, 20)
    marker = free[len(free) // 2]
    cut = gpu.stream(PROMPT, 20, stop=marker)
    assert marker not in cut.text and cut.text == free[: free.index(marker)] and cut.finish_reason == "stop" and cut.buffer_text == cut.text
    assert gpu.generate(PROMPT, 20, stop="☃☃") == free and gpu.generate(PROMPT, 20, stop=[""]) == free
    two = free[len(free) // 2: len(free) // 2 + 2]
    assert gpu.generate(PROMPT, 20, stop=[two, "☃"]) == free[: free.index(two)]  # a stop sequence that arrives in two pieces
    # the window: 64 positions; a prompt that fills it leaves room for exactly one more token
    ids = tok.encode(PROMPT, add_bos=True)
    s = gpu.stream(PROMPT, 100)
    want, out, reason = _oracle_text(cpu, tok, PROMPT, 100)
    assert s.text == want and s.finish_reason == reason and s.n_tokens == len(out) <= 64 - len(ids) + 1
    with pytest.raises(QuintritError) as e:
        gpu.generate("x" * 10000, 5)
    assert e.value.code == 11
    for kw in ({"temperature": -1.0}, {"temperature": float("nan")}, {"top_p": 0.0}, {"top_p": 1.5}):
        with pytest.raises(QuintritError) as e:
            gpu.generate(PROMPT, 5, **kw)
        assert e.value.code == 2
    with pytest.raises(QuintritError) as e:
        gpu.logits([5, 1000])
    assert e.value.code == 2
    with pytest.raises(QuintritError) as e:
        gpu.logits(list(range(65)))
    assert e.value.code == 11
    gpu.reset()
    assert gpu.position == 0
    assert gpu.generate(PROMPT, 20) == free  # the session is usable after every error


def test_a_prompt_that_begins_like_the_cached_conversation_is_ingested_from_the_first_difference(cpu, tok):
    """Prefix reuse (quintrit-runtime/src/engine.rs:700-727): the text is what a fresh session gives, and the count of prompt tokens that
    were found cached is reported."""
    m = Model.load(TINY, device="cuda")
    first = m.generate(PROMPT, 6)
    assert m.reused_tokens() == 0
    n_prompt = len(tok.encode(PROMPT, add_bos=True))
    again = m.generate(PROMPT, 6)  # the whole prompt is cached; its last token is computed again (its logits start the generation)
    assert again == first == _oracle_text(cpu, tok, PROMPT, 6)[0] and m.reused_tokens() == n_prompt - 1
    longer = PROMPT + " and the dog"
    assert m.generate(longer, 5) == _oracle_text(cpu, tok, longer, 5)[0]
    assert m.reused_tokens() >= n_prompt  # the prompt (and a generated token only if the new text happens to continue like it)
    other = "the cat ran"
    common = 0
    a, b = tok.encode(longer, add_bos=True), tok.encode(other, add_bos=True)
    while common < min(len(a), len(b)) and a[common] == b[common]:
        common += 1
    assert m.generate(other, 5, temperature=0.8, seed=3) == _oracle_text(cpu, tok, other, 5, temperature=0.8, top_k=40, top_p=0.9, seed=3)[0]
    assert m.reused_tokens() >= min(common, len(b) - 1) > 0
    m.generate_tokens(tok.encode(PROMPT, add_bos=True), 3)  # the loop runs on the device: the host's record of the cache is dropped
    assert m.generate(PROMPT, 6) == first and m.reused_tokens() == 0
    m.close()


def test_a_session_in_use_is_busy_for_other_threads(gpu):
    started, release, seen = threading.Event(), threading.Event(), []

    def on_piece(_piece):
        started.set()
        release.wait(10)
        return False

    t = threading.Thread(target=lambda: seen.append(gpu.stream(PROMPT, 3, on_piece=on_piece).text))
    t.start()
    assert started.wait(30)
    si = _SessionInfo(struct_size=C.sizeof(_SessionInfo))
    rc = gpu._l.quintrit_session_info(gpu._s, C.byref(si))
    release.set()
    t.join(30)
    assert rc == 12 and seen and seen[0] == gpu.generate(PROMPT, 3)  # QUINTRIT_ERR_BUSY; the generation itself was not disturbed


def test_context_option_and_sessions_of_their_own(cpu, tok):
    m = Model.load(TINY, device="cuda:0", context=32)
    assert m.context_window == 32 and m.context_length == 64
    want, out, reason = _oracle_text(oracle.Model({**cpu.spec, "ctx": 32}), tok, PROMPT, 40)
    s = m.stream(PROMPT, 40)
    assert (s.text, s.finish_reason) == (want, reason)
    m.close()
    with pytest.raises(QuintritError) as e:
        Model.load(TINY, device="cuda:99")
    assert e.value.code in (2, 15)
    with pytest.raises(QuintritError) as e:
        Model.load(TINY, device="cpu")
    assert e.value.code == 2


def test_format_level_conversion_on_the_device():
    spec = gguf_model.model_spec(TINY)
    with GgufFile(TINY) as f:
        planar, rows, cols, scale = f.convert_tensor("blk.1.ffn_down.weight")
        assert (rows, cols) == (128, 256) and scale == np.float32(0.05)
        assert np.array_equal(planar, spec["weights"][7 + 6].reshape(-1))


def _synth_like_the_reference_c_tests(path):
    """A model shaped like the one the reference's C tests write (quintrit-c/tests/common/synth.rs:12-22, 191-250): hidden 128,
    FFN 256, 2 layers, 4 / 2 heads, 264 tokens (bytes, <s>, </s>, six fillers), no merges, BOS 256, EOS 257, context 48."""
    spec = synth.make_model(0, False, 128, 256, 2, 4, 2, 32, 264, 48, 10000.0, 1e-5, config=9)
    shapes = [(128, 128), (64, 128), (64, 128), (128, 128), (256, 128), (256, 128), (128, 256)]
    trits = [synth.trits(synth.seed_for(9, l, p, 0), r * c).reshape(r, c) for l in range(2) for p, (r, c) in enumerate(shapes)]
    table, n = {}, 0
    for b in range(256):  # the published byte-to-character table of byte-level BPE vocabularies
        keep = 0x21 <= b <= 0x7E or 0xA1 <= b <= 0xAC or 0xAE <= b <= 0xFF
        table[b] = chr(b) if keep else chr(256 + n)
        n += 0 if keep else 1
    tokens = [table[b] for b in range(256)] + ["<s>", "</s>"] + [f"<f{i}>" for i in range(6)]
    tokenizer = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": [], "tokenizer.ggml.bos_token_id": 256,
                 "tokenizer.ggml.eos_token_id": 257, "tokenizer.ggml.add_bos_token": True}
    gguf_io.write_model_gguf(path, spec, trits, gguf_io.GGML_I2_S, extra_metadata=tokenizer)


def test_a_qwen3_file_loads_with_its_head_norms_and_the_chatml_prompt(tmp_path):
    """general.architecture "qwen3": NEOX RoPE, blk.N.attn_q_norm / attn_k_norm applied to every head before it
    (config.rs:278-279, 424, 465; engine.rs:480), ChatML with an empty thinking block as the chat prompt (engine.rs:70-87)."""
    spec = synth.make_model(2, True, 128, 256, 2, 4, 2, 32, 264, 48, 10000.0, 1e-6, config=13, random_norms=True)
    shapes = [(128, 128), (64, 128), (64, 128), (128, 128), (256, 128), (256, 128), (128, 256)]
    trits = [synth.trits(synth.seed_for(13, l, p, 0), r * c).reshape(r, c) for l in range(2) for p, (r, c) in enumerate(shapes)]
    rng = np.random.default_rng(13)
    spec["block_scales"] = [rng.uniform(0.5, 2.0, r * c // 64).astype(np.float16).astype(np.float32) for _ in range(2) for r, c in shapes]
    spec["qk_norms"] = [rng.uniform(0.5, 1.5, 32).astype(np.float32) for _ in range(4)]
    tokens = [chr(0x100 + b) for b in range(256)] + ["<s>", "</s>"] + [f"<f{i}>" for i in range(6)]
    tokenizer = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": [], "tokenizer.ggml.bos_token_id": 256,
                 "tokenizer.ggml.eos_token_id": 257, "tokenizer.ggml.add_bos_token": True}
    path = tmp_path / "qwen3.gguf"
    gguf_io.write_model_gguf(path, spec, trits, gguf_io.GGML_Q2_0, architecture="qwen3", extra_metadata=tokenizer)
    m = Model.load(str(path), device="cuda")
    assert m.architecture == "qwen3"
    msgs = [{"role": "system", "content": "Be brief."}, {"role": " User ", "content": "hi"}, {"role": "assistant", "content": "hello"},
            {"role": "tool", "content": "x"}]
    assert m.format_chat(msgs) == ("<|im_start|>system\nBe brief.<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\nhello<|im_end|>\n"
                                   "<|im_start|>user\nx<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n")
    m.close()
    from quintrit_b200 import api

    dec, ref = api.Decoder.open(str(path)), oracle.Model(spec)
    for pos, t in enumerate(synth.prompt_tokens(3, 12, 264)):
        want = ref.forward(int(t), pos)
        got, greedy = dec.forward(int(t), pos)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), pos
        assert greedy == oracle.argmax(want)
    dec.free()


def _run_acceptance(tmp_path, model, prompt):
    exe = tmp_path / "runtime_acceptance"
    lib_dir = os.path.join(ROOT, "quintrit_b200")
    subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), "-o", str(exe),
                    os.path.join(ROOT, "tests", "c", "runtime_acceptance.c"), "-L", lib_dir, "-lquintrit_b200", f"-Wl,-rpath,{lib_dir}"], check=True)
    r = subprocess.run([str(exe), str(model), prompt], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    facts = dict(line.split("=", 1) for line in r.stdout.splitlines() if "=" in line and line.split("=", 1)[0].isupper())
    return r.stdout, facts


def test_c_program_against_the_runtime_header(tmp_path, cpu, tok):
    out, facts = _run_acceptance(tmp_path, TINY, PROMPT)
    assert "runtime acceptance passed" in out
    ids = tok.encode(PROMPT, add_bos=True)
    assert [int(x) for x in facts["PROMPT_IDS"].split(",")] == ids
    assert bytes.fromhex(facts["GREEDY_HEX"]).decode() == _oracle_text(cpu, tok, PROMPT, 10)[0]
    assert bytes.fromhex(facts["SAMPLED_HEX"]).decode() == _oracle_text(cpu, tok, PROMPT, 10, temperature=0.8, top_k=40, top_p=0.9, seed=3)[0]


def test_c_program_on_a_model_like_the_reference_c_tests_write(tmp_path):
    path = tmp_path / "c_test_model.gguf"
    _synth_like_the_reference_c_tests(path)
    prompt = "<|user|>\nHello there\n<|assistant|>\n"  # the prompt of the reference's C test: one token per byte plus BOS
    out, facts = _run_acceptance(tmp_path, path, prompt)
    ids = [int(x) for x in facts["PROMPT_IDS"].split(",")]
    assert ids == [256] + list(prompt.encode())
    cpu, tok = oracle.Model(gguf_model.model_spec(path)), Tokenizer(path)
    want, _ = sampler.generate(cpu, ids, 10, eos=257)
    assert bytes.fromhex(facts["GREEDY_HEX"]).decode() == "".join(tok.decode_pieces(want))
