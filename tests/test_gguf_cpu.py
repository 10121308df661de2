"""The GGUF reader on the host (no GPU): the directory the library parses from a synthetic file must be what the writer put
there, with the hyperparameter derivation and the error classes of the reference
(rust/crates/quintrit-runtime/src/config.rs:257-455; rust/crates/quintrit-c/src/gguf_check.rs:14-28: a path that is not a
regular file is an I/O error, a malformed file a format error)."""
import struct

import numpy as np
import pytest

import quintrit_b200 as q
from quintrit_b200 import gguf_io, synth


def _tiny(arch=0, **kw):
    spec = synth.make_model(arch, False, 256, 512, 2, 4, 2, 64, 300, 512, 500000.0, 1e-5, config=5, random_norms=True, **kw)
    shapes = [(256, 256), (128, 256), (128, 256), (256, 256), (512, 256), (512, 256), (256, 512)]
    trits = [synth.trits(synth.seed_for(5, l, p, 0), r * c).reshape(r, c) for l in range(2) for p, (r, c) in enumerate(shapes)]
    return spec, trits


def test_directory_and_hyperparameters_round_trip(tmp_path):
    spec, trits = _tiny()
    path = tmp_path / "tiny.gguf"
    gguf_io.write_model_gguf(path, spec, trits, gguf_io.GGML_I2_S)
    d = q.gguf_describe(path)
    assert d["version"] == "3" and d["architecture"] == "llama"
    assert [int(d[k]) for k in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads", "num_kv_heads", "head_dim",
                                "rope_dims", "context_length")] == [300, 256, 512, 2, 4, 2, 64, 64, 512]
    assert d["tied"] == "0" and d["f32_values"] == "0"
    assert np.float32(d["rms_norm_eps"]) == np.float32(1e-5) and np.float32(d["rope_theta"]) == np.float32(500000.0)
    by_name = {t["name"]: t for t in d["tensors"]}
    assert len(by_name) == 1 + 2 * 9 + 2 and all(t["inside_file"] for t in d["tensors"])
    assert by_name["token_embd.weight"] == {"name": "token_embd.weight", "inside_file": True, "type": 1, "shape": (256, 300), "bytes": 300 * 256 * 2}
    assert by_name["blk.1.ffn_down.weight"]["type"] == 36 and by_name["blk.1.ffn_down.weight"]["shape"] == (512, 256)
    assert by_name["blk.1.ffn_down.weight"]["bytes"] == 256 * 512 // 4
    assert by_name["blk.0.attn_norm.weight"]["type"] == 0 and by_name["blk.0.attn_norm.weight"]["bytes"] == 1024


def test_defaults_tied_head_and_numerics(tmp_path):
    spec, trits = _tiny(tied=True)
    spec["scales"] = np.float32(np.float16(spec["scales"]))
    path = tmp_path / "tq.gguf"
    gguf_io.write_model_gguf(path, spec, trits, gguf_io.GGML_TQ2_0)
    d = q.gguf_describe(path)
    assert d["tied"] == "1" and d["f32_values"] == "1"  # no output.weight; no I2_S tensor -> FP32 accumulators
    # a file with nothing but an architecture takes the reference's defaults (config.rs:296-353)
    bare = tmp_path / "bare.gguf"
    gguf_io.write_gguf(bare, {"general.architecture": "llama"}, [])
    d = q.gguf_describe(bare)
    assert [int(d[k]) for k in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads", "num_kv_heads", "head_dim",
                                "context_length")] == [128256, 2560, 6912, 30, 20, 5, 128, 4096]
    # without <arch>.vocab_size and without an embedding the tokenizer's token list gives the vocabulary (config.rs:293-304)
    toks = tmp_path / "toks.gguf"
    gguf_io.write_gguf(toks, {"general.architecture": "qwen2", "tokenizer.ggml.tokens": [f"t{i}" for i in range(77)]}, [])
    assert q.gguf_describe(toks)["vocab_size"] == "77"
    # per-layer arrays give their maximum (config.rs:502-512)
    arr = tmp_path / "arr.gguf"
    gguf_io.write_gguf(arr, {"general.architecture": "llama", "llama.attention.head_count_kv": [2, 8, 4], "llama.embedding_length": 512,
                             "llama.attention.head_count": 8}, [])
    d = q.gguf_describe(arr)
    assert d["num_kv_heads"] == "8" and d["head_dim"] == "64"


def test_qwen_files_name_their_architecture_and_carry_head_norms(tmp_path):
    """general.architecture "qwen2" / "qwen3" (config.rs:278-279, 464-467): read like any other file; a qwen3 file holds
    blk.N.attn_q_norm / attn_k_norm of head_dim values (validate.rs:250-251), which the CPU oracle's reader hands on."""
    from oracle import gguf_model

    spec, trits = _tiny(arch=2)
    rng = np.random.default_rng(8)
    spec["qk_norms"] = [rng.uniform(0.5, 1.5, 64).astype(np.float32) for _ in range(4)]
    path = tmp_path / "qwen3.gguf"
    gguf_io.write_model_gguf(path, spec, trits, gguf_io.GGML_I2_S, architecture="qwen3")
    d = q.gguf_describe(path)
    assert d["architecture"] == "qwen3" and int(d["head_dim"]) == 64
    by_name = {t["name"]: t for t in d["tensors"]}
    assert by_name["blk.1.attn_k_norm.weight"]["shape"] == (64,) and by_name["blk.0.attn_q_norm.weight"]["type"] == 0
    got = gguf_model.model_spec(path)
    assert got["arch"] == 2 and all(np.array_equal(a, b) for a, b in zip(got["qk_norms"], spec["qk_norms"]))
    plain = tmp_path / "qwen2.gguf"
    gguf_io.write_model_gguf(plain, {k: v for k, v in spec.items() if k != "qk_norms"}, trits, gguf_io.GGML_I2_S, architecture="qwen2")
    got = gguf_model.model_spec(plain)
    assert got["arch"] == 2 and "qk_norms" not in got and q.gguf_describe(plain)["architecture"] == "qwen2"


def test_error_classes(tmp_path):
    def code(path):
        with pytest.raises(q.QuintritError) as e:
            q.gguf_describe(path)
        return e.value.code

    assert code(tmp_path / "missing.gguf") == 7          # QUINTRIT_ERR_IO
    assert code(tmp_path) == 7                           # a directory is not a regular file
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    assert code(bad) == 8                                # QUINTRIT_ERR_FORMAT: wrong magic
    bad.write_bytes(b"GGUF" + struct.pack("<IQQ", 1, 0, 0))
    assert code(bad) == 8                                # version 1
    bad.write_bytes(b"GG")
    assert code(bad) == 8                                # too short
    spec, trits = _tiny()
    good = tmp_path / "good.gguf"
    gguf_io.write_model_gguf(good, spec, trits, gguf_io.GGML_I2_S)
    raw = good.read_bytes()
    bad.write_bytes(raw[:200])                           # directory cut off in the middle
    assert code(bad) == 8
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(raw[: len(raw) // 2])                # directory intact, payloads missing: reported per tensor
    d = q.gguf_describe(cut)
    assert not all(t["inside_file"] for t in d["tensors"])
    moe = tmp_path / "moe.gguf"
    gguf_io.write_gguf(moe, {"general.architecture": "qwen35"}, [])
    assert code(moe) == 6                                # QUINTRIT_ERR_UNSUPPORTED
    odd = tmp_path / "odd.gguf"
    gguf_io.write_gguf(odd, {"general.architecture": "llama", "llama.attention.key_length": 63}, [])
    assert code(odd) == 10                               # QUINTRIT_ERR_MODEL
