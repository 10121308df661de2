"""Test infrastructure: reads a GGUF file in plain Python and hands its model to the CPU oracle.

Independent of the library's C++ reader (quintrit_b200/csrc/gguf.hpp), so that the two check each other. Follows the
published GGUF layout and the reference's reading of it: rust/crates/quintrit-format/src/gguf.rs:190-358 (directory,
payload views, the f32 scale behind an I2_S payload), rust/crates/quintrit-runtime/src/config.rs:257-455
(hyperparameters, defaults, I2_S files use the F16-accumulator attention) and quintrit-runtime/src/gpu.rs:183-260
(which tensors a decoder needs). Only tests may import this module.
"""
from __future__ import annotations

import struct

import numpy as np

import oracle

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}
F32, F16, BF16, TQ1_0, TQ2_0, I2_S, Q2_0 = 0, 1, 30, 34, 35, 36, 42
VELUREX = 0x5156  # not a GGML type: planar velurex rows in a pre-transcoded container (quintrit_b200/container.py)


class _Cursor:
    def __init__(self, blob: bytes):
        self.b, self.i = blob, 0

    def take(self, fmt: str):
        v = struct.unpack_from(fmt, self.b, self.i)
        self.i += struct.calcsize(fmt)
        return v[0] if len(v) == 1 else v

    def string(self) -> str:
        n = self.take("<Q")
        s = self.b[self.i:self.i + n].decode("utf-8", errors="surrogateescape")
        self.i += n
        return s

    def value(self, t: int):
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.take("<I"), self.take("<Q")
            return [self.value(et) for _ in range(n)]
        v = self.take(_SCALAR[t])
        return bool(v) if t == 7 else v


def read_gguf(path):
    """(version, metadata dict, tensors dict name -> (ggml shape innermost first, type id, offset), data section as bytes)."""
    blob = open(path, "rb").read()
    c = _Cursor(blob)
    assert blob[:4] == b"GGUF"
    c.i = 4
    version, n_tensors, n_kv = c.take("<I"), c.take("<Q"), c.take("<Q")
    meta = {}
    for _ in range(n_kv):
        k = c.string()
        meta[k] = c.value(c.take("<I"))
    tensors = {}
    for _ in range(n_tensors):
        name = c.string()
        rank = c.take("<I")
        shape = [c.take("<Q") for _ in range(rank)]
        t, off = c.take("<I"), c.take("<Q")
        tensors[name] = (shape, t, off)
    align = int(meta.get("general.alignment", 32))
    start = (c.i + align - 1) // align * align
    return version, meta, tensors, memoryview(blob)[start:]


def _payload_len(t: int, n: int) -> int:
    return {F32: n * 4, F16: n * 2, BF16: n * 2, I2_S: (n + 3) // 4, TQ1_0: n // 256 * 54, TQ2_0: n // 256 * 66, Q2_0: n // 64 * 18}[t]


def tensor_bytes(tensors, data, name: str, extra: int = 0) -> np.ndarray:
    shape, t, off = tensors[name]
    n = int(np.prod(shape))
    return np.frombuffer(bytes(data[off:off + _payload_len(t, n) + extra]), np.uint8)


def ternary_tensor(tensors, data, name: str):
    """(trits (rows, cols) int8, per-tensor scale float32) of an I2_S, TQ1_0 or TQ2_0 tensor."""
    shape, t, off = tensors[name]
    cols, rows = shape
    if t == VELUREX:  # a pre-transcoded container's tensor: planar velurex rows, the f32 scale behind them
        nbytes = rows * ((cols + 159) // 160) * 32
        raw = np.frombuffer(bytes(data[off:off + nbytes + 4]), np.uint8)
        return oracle.unpack_planar(raw[:-4], rows, cols), np.frombuffer(raw[-4:].tobytes(), np.float32)[0]
    if t == I2_S:
        raw = tensor_bytes(tensors, data, name, extra=4)
        scale = np.frombuffer(raw[-4:].tobytes(), np.float32)[0]
        return oracle.decode_i2_s(raw[:-4], rows, cols), scale
    raw = tensor_bytes(tensors, data, name)
    scale = oracle.uniform_block_scale(t, raw)
    assert scale is not None, f"{name}: block scales differ"
    return (oracle.decode_tq1_0 if t == TQ1_0 else oracle.decode_tq2_0)(raw, rows, cols), np.float32(scale)


def model_spec(path, ctx: int | None = None) -> dict:
    """The model of a GGUF file as oracle.Model takes it (per-tensor ternary projections, F16 or BF16 tables)."""
    _, meta, tensors, data = read_gguf(path)
    a = meta.get("general.architecture", "bitnet-b1.58")
    arch = 1 if a in ("bitnet-b1.58", "bitnet") else 2 if a in ("qwen2", "qwen3") else 0  # config.rs:419-424, 464-467
    g = lambda k, d: meta.get(f"{a}.{k}", d)  # noqa: E731
    hidden, inter, layers = g("embedding_length", 2560), g("feed_forward_length", 6912), g("block_count", 30)
    heads, kv_heads = g("attention.head_count", 20), g("attention.head_count_kv", 5)
    head_dim = g("attention.key_length", hidden // heads)
    vocab = g("vocab_size", tensors["token_embd.weight"][0][1])
    ctx_train = g("context_length", 4096)
    want = min(ctx_train, ctx or 4096, 7936)
    want = want // 256 * 256 if want >= 256 else want
    table_t = tensors["token_embd.weight"][1]
    tab = lambda name: np.frombuffer(tensor_bytes(tensors, data, name).tobytes(), np.uint16).copy()  # noqa: E731
    f32 = lambda name: np.frombuffer(tensor_bytes(tensors, data, name).tobytes(), np.float32).copy()  # noqa: E731
    weights, scales, norms, qk_norms = [], [], [], []
    qd, kvd = heads * head_dim, kv_heads * head_dim
    shapes = [(qd, hidden), (kvd, hidden), (kvd, hidden), (hidden, qd), (inter, hidden), (inter, hidden), (hidden, inter)]
    for l in range(layers):
        for k, nm in enumerate(("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")):
            trits, s = ternary_tensor(tensors, data, f"blk.{l}.{nm}.weight")
            assert trits.shape == shapes[k]
            weights.append(oracle.pack_planar(trits, *shapes[k]))
            scales.append(s)
        for k, nm in enumerate(("attn_norm", "ffn_norm", "attn_sub_norm", "ffn_sub_norm")):
            norms.append(f32(f"blk.{l}.{nm}.weight") if (k < 2 or arch == 1) else None)
        if a == "qwen3":  # engine.rs:480: query and key head norms
            qk_norms += [f32(f"blk.{l}.attn_q_norm.weight"), f32(f"blk.{l}.attn_k_norm.weight")]
    return {
        **({"qk_norms": qk_norms} if qk_norms else {}),
        "arch": arch, "f32_values": bool(meta["quintrit_b200.f32_values"]) if "quintrit_b200.f32_values" in meta else not any(t == I2_S for _, t, _ in tensors.values()), "hidden": hidden, "inter": inter, "layers": layers,
        "q_heads": heads, "kv_heads": kv_heads, "head_dim": head_dim, "vocab": vocab, "ctx": want, "rope_dims": g("rope.dimension_count", head_dim),
        "eps": float(g("attention.layer_norm_rms_epsilon", 1e-5)), "rope_theta": float(g("rope.freq_base", 500000.0)),
        "embed": tab("token_embd.weight"), "lm_head": tab("output.weight") if "output.weight" in tensors else None,
        "out_norm": f32("output_norm.weight"), "weights": weights, "scales": np.array(scales, np.float32), "norms": norms,
        "bf16_tables": table_t == BF16,
    }
