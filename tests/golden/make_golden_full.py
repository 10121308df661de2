"""Generates the full-size greedy-decoding fixtures with the CPU oracle (run on a CPU box; needs no GPU).

    python tests/golden/make_golden_full.py --model falcon3_10b --variant i2_s            # 40 layers, 1024 + 512 tokens
    python tests/golden/make_golden_full.py --model bitnet_2b --variant i2_s --tables bf16 # 30 layers, 512 + 256 tokens

For one named model (quintrit_b200.synth.full_model: every weight machine-independent) the oracle ingests the seeded
prompt token by token and then decodes greedily; the file keeps the generated token ids, the margin between the best
and the second-best logit at every generated step (how much room a non-bit-exact device would have) and the logits
of the last step. tests/test_full_parity_gpu.py loads the same model on the GPU from a synthetic GGUF in every encoding
that shares the variant's arithmetic and compares. Variants: i2_s (FP16-accumulator attention), tq (TQ1_0 and TQ2_0
files: tensor scales exact in F16, FP32 accumulators), q2_0 (block-scaled projections).

The model is built by the oracle library's threaded generators (oracle.full_model: the same values as
quintrit_b200.synth.full_model, tests/test_synth.py), which takes about a minute for the 9.5 G weights of the Falcon3-10B shape.
"""
import argparse
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from quintrit_b200 import synth  # noqa: E402

SIZES = {"falcon3_10b": (1024, 512), "bitnet_2b": (512, 256)}


def fixture_name(model: str, variant: str, tables: str, layers: int | None = None) -> str:
    return f"full_{model}_{variant}_{tables}" + (f"_l{layers}" if layers else "") + ".npz"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=sorted(SIZES), required=True)
    ap.add_argument("--variant", choices=["i2_s", "tq", "q2_0"], default="i2_s")
    ap.add_argument("--tables", choices=["f16", "bf16"], default="f16")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (quick checks; the file name says so)")
    ap.add_argument("--prompt", type=int, default=None)
    ap.add_argument("--new", type=int, default=None)
    ap.add_argument("--out-dir", default=os.path.dirname(os.path.abspath(__file__)))
    args = ap.parse_args()
    P, G = SIZES[args.model]
    P, G = args.prompt or P, args.new or G
    ctx = (P + G + 255) // 256 * 256
    t0 = time.time()
    spec = oracle.full_model(args.model, args.variant, ctx, bf16_tables=args.tables == "bf16", layers=args.layers)
    print(f"model ready after {time.time() - t0:.0f} s", flush=True)
    m = oracle.Model(spec)
    prompt = synth.prompt_tokens(spec_config(args.model), P, spec["vocab"])
    t1 = time.time()
    logits = None
    for pos, tok in enumerate(prompt):
        logits = m.forward(int(tok), pos)
        if pos % 64 == 0:
            print(f"prompt {pos}/{P} {time.time() - t1:.0f} s", flush=True)
    tokens, margins = np.zeros(G, np.uint32), np.zeros(G, np.float32)
    for i in range(G):
        top2 = np.partition(logits, -2)[-2:]
        tokens[i] = oracle.argmax(logits)
        margins[i] = top2[1] - top2[0]
        if i + 1 < G:
            logits = m.forward(int(tokens[i]), P + i)
        if i % 64 == 0:
            print(f"decode {i}/{G} {time.time() - t1:.0f} s", flush=True)
    # the logits that chose tokens[G - 1] are those of position P + G - 2
    out = os.path.join(args.out_dir, fixture_name(args.model, args.variant, args.tables, args.layers))
    np.savez_compressed(out, tokens=tokens, margins=margins, last_logits=logits, prompt_len=np.int64(P), layers=np.int64(spec["layers"]),
                        ctx=np.int64(ctx), oracle_seconds=np.float64(time.time() - t1))
    print(f"wrote {out}: {G} tokens in {time.time() - t1:.0f} s, smallest margin {margins.min():.3g}", flush=True)


def spec_config(model: str) -> int:
    return synth.full_dims(model)["config"]


if __name__ == "__main__":
    main()
