"""The pre-transcoded container (quintrit_b200/container.py) on the host: every metadata entry and dense tensor of the source file is kept,
the ternary projections become planar velurex rows with their scale, and the oracle reads the same model from either file. The transcoder is
the oracle's here (the library's runs on the GPU: tests/test_container_gpu.py)."""
import os

import numpy as np

import oracle
from oracle import gguf_model
from quintrit_b200 import container
from quintrit_b200.runtime import Tokenizer

TINY = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_tiny_model.gguf")


def _oracle_transcoder(path):
    _, _, tensors, data = gguf_model.read_gguf(path)

    def transcode(name):
        trits, scale = gguf_model.ternary_tensor(tensors, data, name)
        rows, cols = trits.shape
        return oracle.pack_planar(trits, rows, cols), rows, cols, scale

    return transcode


def test_container_holds_the_same_model(tmp_path):
    dst = tmp_path / "tiny.qtb.gguf"
    stats = container.convert(TINY, dst, transcode=_oracle_transcoder(TINY))
    assert stats["converted"] == 2 * 7 and stats["tensors"] == len(gguf_model.read_gguf(TINY)[2])
    assert stats["container_bytes"] == os.path.getsize(dst)  # (this model's 128-column rows fill one 160-trit block: no smaller than 2 bits a weight)
    _, meta_a, tensors_a, _ = gguf_model.read_gguf(TINY)
    _, meta_b, tensors_b, _ = gguf_model.read_gguf(dst)
    assert {k: v for k, v in meta_b.items() if not k.startswith("quintrit_b200.")} == meta_a
    assert meta_b["quintrit_b200.container_version"] == 1 and meta_b["quintrit_b200.f32_values"] == 0  # an I2_S file: F16-accumulator attention
    assert list(tensors_a) == list(tensors_b)
    assert all(tensors_b[n][1] == (container.GGML_VELUREX if tensors_a[n][1] == gguf_model.I2_S else tensors_a[n][1]) for n in tensors_a)
    a, b = gguf_model.model_spec(TINY), gguf_model.model_spec(dst)
    assert a.keys() == b.keys()
    for k in a:
        if k == "weights":
            assert all(np.array_equal(x, y) for x, y in zip(a[k], b[k]))
        elif k == "norms":
            assert all((x is None and y is None) or np.array_equal(x, y) for x, y in zip(a[k], b[k]))
        elif isinstance(a[k], np.ndarray):
            assert np.array_equal(a[k], b[k]), k
        else:
            assert a[k] == b[k], k
    tok_a, tok_b = Tokenizer(TINY), Tokenizer(str(dst))  # the tokenizer's metadata travels with the container
    assert tok_a.encode("the cat sat", add_bos=True) == tok_b.encode("the cat sat", add_bos=True)
    # a container has no I2_S / TQ tensors left to convert
    again = container.convert(dst, tmp_path / "again.gguf", transcode=lambda name: (_ for _ in ()).throw(AssertionError(name)))
    assert again["converted"] == 0
