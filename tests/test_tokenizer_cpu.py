"""The byte-level BPE tokenizer of the library (host only) against answers of the Hugging Face `tokenizers` library configured
as the reference configures it (rust/crates/quintrit-runtime/src/tokenizer.rs:82-146, 215-293), stored in
tests/golden/tokenizer_vectors.json.gz by tests/golden/make_golden_tokenizer.py, and on the vocabulary of the reference's own
tiny test model (tests/golden/ref_tiny_model.gguf, written by the reference's gguf_builder.py)."""
import gzip
import json
import os

import pytest

from quintrit_b200 import gguf_io
from quintrit_b200.api import QuintritError
from quintrit_b200.runtime import Tokenizer

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def vectors():
    with gzip.open(os.path.join(GOLDEN, "tokenizer_vectors.json.gz"), "rt", encoding="utf-8") as f:
        return json.load(f)


def _tokenizer_file(tmp_path, v, kind, **extra):
    meta = {"general.architecture": "llama", "tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": v["tokens"], "tokenizer.ggml.merges": v["merges"],
            "tokenizer.ggml.token_type": v["types"], "tokenizer.ggml.bos_token_id": v["bos"], "tokenizer.ggml.eos_token_id": v["eos"],
            "tokenizer.ggml.add_bos_token": True}
    if v["pre"][kind] is not None:
        meta["tokenizer.ggml.pre"] = v["pre"][kind]
    meta.update(extra)
    path = tmp_path / f"tok_{kind}.gguf"
    gguf_io.write_gguf(path, meta, [])
    return path


@pytest.mark.parametrize("kind", ["default", "gpt2", "llama3", "qwen2"])
def test_encode_and_decode_match_the_library_the_reference_uses(tmp_path, vectors, kind):
    tok = Tokenizer(_tokenizer_file(tmp_path, vectors, kind))
    assert len(tok) == len(vectors["tokens"]) and tok.bos_token_id == vectors["bos"] and tok.eos_token_id == vectors["eos"]
    want = vectors["kinds"][kind]
    bad = []
    for text, ids, dec in zip(vectors["texts"], want["ids"], want["decoded"]):
        got = tok.encode(text)
        if got != ids:
            bad.append((text, got, ids))
            continue
        assert tok.decode(ids) == dec, text
    assert not bad, f"{len(bad)} of {len(vectors['texts'])} texts tokenize differently; first: {bad[0]}"


def test_streaming_pieces_never_split_a_character(tmp_path, vectors):
    tok = Tokenizer(_tokenizer_file(tmp_path, vectors, "gpt2"))
    for text in ("日本語 🙂 naïve ☃☃", "plain ascii", "é🚀"):
        ids = tok.encode(text)
        pieces = tok.decode_pieces(ids)
        assert len(pieces) == len(ids) + 1 and "".join(pieces) == text and "�" not in "".join(pieces)
    ids = tok.encode("🎉🎉")  # not in the training text: four byte tokens each
    assert len(ids) > 2 and "" in tok.decode_pieces(ids)  # tokens that end inside a character are held back
    assert tok.decode_pieces([]) == [""]


def test_bos_rules(tmp_path, vectors):
    tok = Tokenizer(_tokenizer_file(tmp_path, vectors, "gpt2"))
    ids = tok.encode("hi", add_bos=True)
    assert ids[0] == tok.bos_token_id and ids[1:] == tok.encode("hi")
    assert tok.encode("<s>hi", add_bos=True)[0] == tok.bos_token_id and tok.encode("<s>hi", add_bos=True).count(tok.bos_token_id) == 1
    # add_bos_token = false: no BOS id at all (config.rs:376-392); absent: by the pre-tokenizer kind
    off = Tokenizer(_tokenizer_file(tmp_path, vectors, "gpt2", **{"tokenizer.ggml.add_bos_token": False}))
    assert off.bos_token_id is None and off.encode("hi", add_bos=True) == off.encode("hi")


def test_the_reference_tiny_vocabulary():
    tok = Tokenizer(os.path.join(GOLDEN, "ref_tiny_model.gguf"))
    assert len(tok) == 261 and tok.bos_token_id == 259 and tok.eos_token_id == 260
    ids = tok.encode("Hello")
    assert ids == [ord(c) for c in "Hello"] and tok.decode(ids) == "Hello"  # bytes are their own ids in this vocabulary
    assert len(tok.encode(" the")) == 1 and len(tok.encode("the")) == 1 and tok.encode("") == [] and tok.decode([]) == ""
    assert tok.encode(" the") == [258] and tok.encode("the") == [257] and tok.encode("th") == [256]
    text = "naïve 日本語 ☃"
    assert tok.decode(tok.encode(text)) == text and len(tok.encode(text)) > len(text)
    assert tok.decode_token(tok.encode("a")[0]) == "a"
    prompt = "<|user|>\nHello there\n<|assistant|>\n"
    assert len(tok.encode(prompt, add_bos=True)) == len(prompt) + 1 - 3  # BOS + one token per byte, except " there" = " the" + "r" + "e"


def test_errors(tmp_path, vectors):
    with pytest.raises(QuintritError) as e:
        Tokenizer(tmp_path / "missing.gguf")
    assert e.value.code == 7
    bare = tmp_path / "bare.gguf"
    gguf_io.write_gguf(bare, {"general.architecture": "llama"}, [])
    with pytest.raises(QuintritError) as e:
        Tokenizer(bare)
    assert e.value.code == 6 and "tokenizer" in str(e.value)
    with pytest.raises(QuintritError) as e:
        Tokenizer(_tokenizer_file(tmp_path, vectors, "gpt2", **{"tokenizer.ggml.pre": "tekken"}))
    assert e.value.code == 6 and "tekken" in str(e.value)
    tok = Tokenizer(_tokenizer_file(tmp_path, vectors, "gpt2"))
    with pytest.raises(QuintritError) as e:
        tok.decode([10_000_000])
    assert e.value.code == 2
    with pytest.raises(TypeError):
        tok.decode("abc")
    with pytest.raises(OverflowError):
        tok.decode([-1])
