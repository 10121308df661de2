"""The committed full-size fixtures are well formed, and the oracle on this machine reproduces the committed one-layer
fixture bit for bit (the fixtures were computed on another machine: this guards the oracle's machine independence -
integer generators, IEEE single operations, the same libm)."""
import glob
import os

import numpy as np

from quintrit_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_fixture_files_are_well_formed():
    files = sorted(glob.glob(os.path.join(GOLDEN, "full_*.npz")))
    assert files, "no full-size fixture is committed"
    for f in files:
        fx = np.load(f)
        model = "falcon3_10b" if "falcon3_10b" in f else "bitnet_2b"
        d = synth.full_dims(model)
        assert fx["tokens"].dtype == np.uint32 and fx["margins"].shape == fx["tokens"].shape and fx["last_logits"].shape == (d["vocab"],)
        assert fx["tokens"].max() < d["vocab"] and (fx["margins"] >= 0).all() and np.isfinite(fx["last_logits"]).all()
        assert int(fx["ctx"]) % 256 == 0 and int(fx["prompt_len"]) + len(fx["tokens"]) <= int(fx["ctx"]) + 1
        if "_l" not in os.path.basename(f).replace("full_", ""):
            assert int(fx["layers"]) == d["layers"]
            assert (int(fx["prompt_len"]), len(fx["tokens"])) == {"falcon3_10b": (1024, 512), "bitnet_2b": (512, 256)}[model]


def test_the_oracle_reproduces_the_one_layer_fixture(oracle):
    fx = np.load(os.path.join(GOLDEN, "full_bitnet_2b_i2_s_f16_l1.npz"))
    P, G = int(fx["prompt_len"]), len(fx["tokens"])
    spec = oracle.full_model("bitnet_2b", "i2_s", int(fx["ctx"]), layers=1)
    m = oracle.Model(spec)
    logits = None
    for pos, tok in enumerate(synth.prompt_tokens(synth.full_dims("bitnet_2b")["config"], P, spec["vocab"])):
        logits = m.forward(int(tok), pos)
    for i in range(G):
        tok = oracle.argmax(logits)
        assert tok == int(fx["tokens"][i])
        if i + 1 < G:
            logits = m.forward(tok, P + i)
    assert np.array_equal(logits.view(np.uint32), fx["last_logits"].view(np.uint32))
