"""A model loaded from its pre-transcoded container (quintrit_b200/container.py, transcoded by the library on the GPU) behaves like the model
loaded from the source file: bit-identical logits, identical text; the container's projections are the planar bytes the oracle packs."""
import os

import numpy as np
import pytest

import oracle
from oracle import gguf_model
from quintrit_b200 import container, gguf_io, synth
from quintrit_b200.runtime import GgufFile, Model

pytestmark = pytest.mark.gpu
TINY = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_tiny_model.gguf")


def test_container_of_the_reference_tiny_model(tmp_path):
    dst = str(tmp_path / "tiny.qtb.gguf")
    stats = container.convert(TINY, dst)
    assert stats["converted"] == 14
    a, b = gguf_model.model_spec(TINY), gguf_model.model_spec(dst)
    assert all(np.array_equal(x, y) for x, y in zip(a["weights"], b["weights"])) and np.array_equal(a["scales"], b["scales"])
    info = GgufFile(dst).tensor("blk.0.attn_q.weight")
    assert info["dtype"] == "VELUREX" and info["dtype_id"] == container.GGML_VELUREX
    src, con = Model.load(TINY, device="cuda"), Model.load(dst, device="cuda")
    prompt = "the cat sat on the mat"
    assert np.array_equal(src.logits(prompt).view(np.uint32), con.logits(prompt).view(np.uint32))
    assert src.generate(prompt, 12) == con.generate(prompt, 12)
    assert src.generate(prompt, 12, temperature=0.8, seed=5) == con.generate(prompt, 12, temperature=0.8, seed=5)
    src.close()
    con.close()


@pytest.mark.parametrize("encoding", [gguf_io.GGML_TQ1_0, gguf_io.GGML_TQ2_0])
def test_container_of_a_model_with_float_accumulator_attention(tmp_path, encoding):
    """TQ files select the F32-accumulator attention (config.rs:425-429); the container records that choice."""
    spec = synth.make_model(0, True, 256, 512, 2, 4, 2, 64, 300, 256, 500000.0, 1e-5, config=61, random_norms=True)
    spec["scales"] = np.float32(np.float16(spec["scales"]))  # the tensor scale is the f16 of every block
    shapes = [(256, 256), (128, 256), (128, 256), (256, 256), (512, 256), (512, 256), (256, 512)]
    trits = [synth.trits(synth.seed_for(61, l, p, 0), r * c).reshape(r, c) for l in range(2) for p, (r, c) in enumerate(shapes)]
    src = str(tmp_path / "m.gguf")
    gguf_io.write_model_gguf(src, spec, trits, encoding=encoding)
    dst = str(tmp_path / "m.qtb.gguf")
    stats = container.convert(src, dst)
    assert stats["converted"] == 14
    assert gguf_model.read_gguf(dst)[1]["quintrit_b200.f32_values"] == 1
    import quintrit_b200 as q

    a, b = q.Decoder.open(src), q.Decoder.open(dst)
    assert a.info()["f32_values"] == b.info()["f32_values"] == 1
    for pos, tok in enumerate(synth.prompt_tokens(4, 9, spec["vocab"])):
        la, ta = a.forward(int(tok), pos)
        lb, tb = b.forward(int(tok), pos)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)) and ta == tb
    a.free()
    b.free()
