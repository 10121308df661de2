"""Test infrastructure: a mixture-of-experts feed-forward block composed of the reference's pieces, for the parity tests of
quintrit_b200_moe_*. The reference has no softmax-routed MoE with ternary SwiGLU experts (its `Moe` is Nemotron-H's: sigmoid router
with a bias, squared-ReLU experts, a shared expert, rust/crates/quintrit-runtime/src/hybrid.rs:798-869), so this block has no
reference run to pin it: parity unpinned. What it is made of, each piece as the reference computes it:
  * the router as a BF16 projection: the input rounded with f32_to_bf16, every row through ggml_vec_dot_bf16 (hybrid.rs:327-333);
  * softmax over the experts (ops.rs:274-298: running maximum, float exponential, sum in double, one multiply);
  * experts by descending probability as std::sort orders them (hybrid.rs:828-831; without ties every sort agrees, and the tests
    draw no ties), the first top_k chosen;
  * their probabilities divided by their sum (added in double, narrowed to float, at least 2^-14: hybrid.rs:833-839);
  * an expert as the dense model's FFN: int8 absmax activations (ops.rs:241-267), exact integer GEMV, one multiply by
    weight_scale / act_scale (layer.rs:123-177), SwiGLU (ops.rs:427-464), the same again for the down projection;
  * the weighted expert outputs added in selection order, the first one assigned (hybrid.rs:847-858).
Only tests, smoke() and the benchmark's checks may import this module.
"""
from __future__ import annotations

import numpy as np

import oracle


def router_probs(x, router_bits, n_experts: int) -> np.ndarray:
    hidden = x.size
    xb = oracle.f32_to_bf16_bits(x)
    rows = np.asarray(router_bits, np.uint16).reshape(n_experts, hidden)
    logits = np.array([oracle.vec_dot_bf16(rows[e], xb) for e in range(n_experts)], np.float32)
    e = oracle.expf_restated(logits - logits.max())
    total = 0.0
    for v in e:
        total += float(v)
    return e * np.float32(1.0 / total) if total > 0 else e


def select(probs, top_k: int):
    order = sorted(range(probs.size), key=lambda i: (-float(probs[i]), i))  # no ties in the tests: any sort gives this order
    chosen = order[:top_k]
    w = probs[chosen].astype(np.float32)
    total = 0.0
    for v in w:
        total += float(v)
    s = max(np.float32(total), np.float32(6.103515625e-5))
    return np.array(chosen, np.uint32), (w / s).astype(np.float32)


def expert(x, gate_up_planar, down_planar, hidden: int, inter: int, ws_gate, ws_up, ws_down) -> np.ndarray:
    a, s = oracle.quantize_int8(x)
    acc = oracle.gemv_planar(gate_up_planar, 2 * inter, hidden, a)
    gate, up = oracle.rescale(acc[:inter], ws_gate, s), oracle.rescale(acc[inter:], ws_up, s)
    v = oracle.swiglu(gate, up)
    a2, s2 = oracle.quantize_int8(v)
    return oracle.rescale(oracle.gemv_planar(down_planar, hidden, inter, a2), ws_down, s2)


def combine(pairs, w) -> np.ndarray:
    """The pairs' results ([top_k][hidden]) weighted and added in selection order, the first one assigned (hybrid.rs:853-857)."""
    out = None
    for i in range(len(w)):
        y = (np.asarray(pairs[i], np.float32) * w[i]).astype(np.float32)
        out = y if i == 0 else (out + y).astype(np.float32)
    return out


def forward(x, router_bits, gate_up, down, scales, hidden: int, inter: int, top_k: int):
    """One token through the block. gate_up[e]: planar rows of the expert's gate rows followed by its up rows; down[e]: planar rows of its
    down projection; scales[e] = (gate, up, down). Returns (output, chosen experts, their weights)."""
    probs = router_probs(np.asarray(x, np.float32), router_bits, len(gate_up))
    chosen, w = select(probs, top_k)
    out = None
    for i, e in enumerate(chosen):
        y = expert(x, gate_up[e], down[e], hidden, inter, *scales[e]) * w[i]
        out = y if i == 0 else (out + y).astype(np.float32)
    return out.astype(np.float32), chosen, w
