"""Test infrastructure: the reference's token sampler and generation loop restated in numpy, for the parity tests of the
text path. Follows rust/crates/quintrit-runtime/src/sampler.rs:43-143 (xorshift64 stream, greedy rule, temperature, stable
descending order, top-k, softmax of ops.rs:274-298 with the float exponential summed in double, nucleus cut, renormalise,
draw) and the loop of rust/crates/quintrit-c/src/runtime.rs:382-520 (BOS in front, EOS or 128009 ends a llama-like model,
the token is fed after it was emitted). Only tests may import this module.
"""
from __future__ import annotations

import numpy as np

import oracle

_M64 = (1 << 64) - 1


class Sampler:
    def __init__(self, temperature: float = 0.0, top_k: int = 1, top_p: float = 1.0, seed: int = 0):
        self.temperature, self.top_k, self.top_p = np.float32(temperature), int(top_k), np.float32(top_p)
        self.state = seed if seed != 0 else 0x5EEDC0DE12345678

    def greedy(self) -> bool:
        return self.temperature <= 0 or self.top_k == 1

    def next_f32(self) -> np.float32:
        x = self.state
        x ^= (x << 13) & _M64
        x ^= x >> 7
        x ^= (x << 17) & _M64
        self.state = x
        return np.float32(np.float32(np.uint64(x)) / np.float32(2.0 ** 64))

    def sample(self, logits: np.ndarray) -> int:
        logits = np.asarray(logits, np.float32)
        if self.greedy():
            return oracle.argmax(logits)
        scaled = logits * (np.float32(1.0) / self.temperature)
        idx = np.arange(scaled.size)
        truncate_k = 0 < self.top_k < scaled.size
        if truncate_k or self.top_p < 1:
            key = scaled.view(np.int32).astype(np.int64)
            key = np.where(key < 0, key ^ 0x7FFFFFFF, key)  # the order of f32::total_cmp
            idx = np.argsort(-key, kind="stable")
        if truncate_k:
            idx = idx[: self.top_k]
        v = scaled[idx]
        e = oracle.expf_restated(v - v.max())  # glibc expf, correctly rounded in all but rare cases, as f32::exp calls it
        total = 0.0
        for x in e:
            total += float(x)
        probs = e * np.float32(1.0 / total) if total > 0 else e
        cutoff = probs.size
        if self.top_p < 1:
            cum = np.float32(0)
            for i, p in enumerate(probs):
                cum = np.float32(cum + p)
                if cum >= self.top_p:
                    cutoff = i + 1
                    break
        probs, idx = probs[:cutoff], idx[:cutoff]
        s = np.float32(0)
        for p in probs:
            s = np.float32(s + p)
        if s > 0:
            probs = probs * np.float32(np.float32(1.0) / s)
        r = self.next_f32()
        acc = np.float32(0)
        for i, p in enumerate(probs):
            acc = np.float32(acc + p)
            if r <= acc or i == probs.size - 1:
                return int(idx[i])
        return int(idx[0])


def generate(model: "oracle.Model", prompt_ids, max_tokens: int, sampler: Sampler | None = None, eos: int | None = None, llama_like: bool = True,
             ctx: int | None = None, pos0: int = 0):
    """Token ids the reference's loop would emit for a prompt given as ids (BOS included by the caller), and the reason it ended."""
    sampler = sampler or Sampler()
    ctx = ctx or model.spec["ctx"]
    logits = None
    pos = pos0
    for t in prompt_ids:
        logits = model.forward(int(t), pos)
        pos += 1
    out, reason = [], "length"
    for _ in range(max_tokens):
        nxt = sampler.sample(logits)
        if (eos is not None and nxt == eos) or (llama_like and nxt == 128009):
            reason = "eos"
            break
        out.append(nxt)
        if pos >= ctx:
            reason = "context"
            break
        logits = model.forward(nxt, pos)
        pos += 1
    return out, reason
