"""Full-size greedy decoding against the committed CPU-oracle fixtures (tests/golden/full_*.npz, made offline by
tests/golden/make_golden_full.py): BitNet-b1.58-2B shape, 30 layers, 512 prompt + 256 greedy tokens, F16 and BF16
tables; Falcon3-10B shape, 40 layers, 1024 + 512 tokens, loaded from a synthetic GGUF file in each of I2_S, TQ1_0, TQ2_0
and Q2_0 and transcoded on the device. The reference holds its GPU engine to its CPU engine the same way at run time
(rust/crates/quintrit-c/tests/engine_gpu.rs:23-100); here the CPU side was run ahead of time. Bar: every generated token
identical and the logits of the last step equal bit for bit."""
import os

import numpy as np
import pytest

import quintrit_b200 as q
from quintrit_b200 import gguf_io, synth

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

CASES = [
    ("bitnet_2b", "i2_s", "f16", gguf_io.GGML_I2_S),
    ("bitnet_2b", "i2_s", "bf16", gguf_io.GGML_I2_S),
    ("falcon3_10b", "i2_s", "f16", gguf_io.GGML_I2_S),
    ("falcon3_10b", "tq", "f16", gguf_io.GGML_TQ2_0),
    ("falcon3_10b", "tq", "f16", gguf_io.GGML_TQ1_0),
    ("falcon3_10b", "q2_0", "f16", gguf_io.GGML_Q2_0),
]


def check_against_fixture(model: str, variant: str, tables: str, encoding: int, workdir, device: int = 0, layers=None) -> dict:
    """Writes the model file, opens it on the GPU, decodes the fixture's sequence and compares. Returns what was checked."""
    import torch

    name = f"full_{model}_{variant}_{tables}" + (f"_l{layers}" if layers else "") + ".npz"
    path = os.path.join(GOLDEN, name)
    if not os.path.exists(path):
        pytest.skip(f"fixture {name} is not committed")
    fx = np.load(path)
    P, G, ctx = int(fx["prompt_len"]), len(fx["tokens"]), int(fx["ctx"])
    file = os.path.join(str(workdir), f"{model}_{encoding}.gguf")
    d = gguf_io.write_full_model_gguf(file, model, encoding, torch.device("cuda", device), ctx, bf16_tables=tables == "bf16", layers=layers)
    torch.cuda.empty_cache()
    try:
        dec = q.Decoder.open(file, context=ctx, device=device)
    finally:
        os.unlink(file)
    try:
        info = dec.info()
        assert info["num_layers"] == int(fx["layers"]) and info["context_length"] == ctx
        assert info["f32_values"] == (0 if variant == "i2_s" else 1) and info["table_dtype"] == (1 if tables == "bf16" else 0)
        prompt = synth.prompt_tokens(d["config"], P, d["vocab"])
        got = dec.generate(prompt, G)
        same = int(np.argmax(np.concatenate([got != fx["tokens"], [True]])))  # index of the first difference
        assert same == G, f"{name}, encoding {encoding}: token {same} of {G} differs (margin there {fx['margins'][same]:.3g})"
        # the logits that chose the last token: position P + G - 2 fed with the token before it (or the last prompt token)
        fed = int(got[G - 2]) if G >= 2 else int(prompt[-1])
        logits, greedy = dec.forward(fed, P + G - 2)
        assert greedy == int(fx["tokens"][-1])
        want = fx["last_logits"]
        bit_exact = bool(np.array_equal(logits.view(np.uint32), want.view(np.uint32)))
        rel = float(np.max(np.abs(logits - want)) / max(np.max(np.abs(want)), 1e-30))
        assert bit_exact, f"{name}: last logits differ, max-abs relative {rel:.3g}"
        return {"fixture": name, "encoding": encoding, "layers": info["num_layers"], "prompt": P, "greedy_tokens_checked": G, "identical": True,
                "logits_bit_exact": bit_exact, "logits_max_rel": rel, "smallest_margin": float(fx["margins"].min()), "single_kernel": info["single_kernel"],
                "ms_per_token": round(dec.time_token(3, 20), 4), "context": P + G - 1}
    finally:
        dec.free()


@pytest.mark.parametrize("model,variant,tables,encoding", CASES)
def test_full_size_sequences_match_the_cpu_oracle(tmp_path, model, variant, tables, encoding):
    check_against_fixture(model, variant, tables, encoding, tmp_path)


def test_reduced_depth_sequence(tmp_path):
    """The one-layer fixture the CPU suite also regenerates (tests/test_full_fixture_cpu.py): a cheap first signal."""
    check_against_fixture("bitnet_2b", "i2_s", "f16", gguf_io.GGML_I2_S, tmp_path, layers=1)
