"""Writers for synthetic GGUF model files and the ternary tensor encodings they hold (numpy, host side).

Used to build seeded random models of any shape without a download: `write_model_gguf` turns a model description (the
dict of `quintrit_b200.synth.make_model`, trits instead of packed bytes) into a file that
`quintrit_b200_decoder_open_gguf` - and the reference's own loader - can read. The container follows the published
GGUF v3 layout; the tensor names and metadata keys are the ones `ModelConfig::from_gguf` and `GpuModel::load` read
(rust/crates/quintrit-runtime/src/config.rs:257-455, gpu.rs:183-260). Encodings: I2_S
(rust/crates/quintrit-format/src/decoders/i2_s.rs:20-67: 128 trits per 32 bytes, plane 0 in bits 6-7, f32 scale behind the
payload), TQ2_0 / TQ1_0 (ggml block layouts, decoders/tq2_0.rs:48-88, tq1_0.rs:51-122, one f16 scale per block), Q2_0
(decoders/q2_0.rs:1-8: f16 scale + 16 code bytes per 64 weights).
"""
from __future__ import annotations

import struct

import numpy as np

GGML_F32, GGML_F16, GGML_BF16, GGML_TQ1_0, GGML_TQ2_0, GGML_I2_S, GGML_Q2_0 = 0, 1, 30, 34, 35, 36, 42
ALIGNMENT = 32


def encode_i2_s(trits, rows: int, cols: int) -> np.ndarray:
    """rows x cols trits (cols a multiple of 128) -> rows * cols / 4 bytes: element j of a 128-block sits in byte j % 32 at
    bits 6 - 2 * (j // 32), code = trit + 1."""
    t = (np.asarray(trits, np.int64).reshape(rows, cols // 128, 4, 32) + 1).astype(np.uint8)
    b = (t[:, :, 0] << 6) | (t[:, :, 1] << 4) | (t[:, :, 2] << 2) | t[:, :, 3]
    return b.reshape(-1)


def encode_tq2_0(trits, d_bits: int = 0x3800) -> np.ndarray:
    """256 trits per block: two groups of 32 bytes, plane l of a group in bits 2l..2l+1, then the f16 scale."""
    t = np.asarray(trits, np.int64).reshape(-1, 2, 4, 32) + 1
    q = (t << (2 * np.arange(4)).reshape(1, 1, 4, 1)).sum(axis=2).astype(np.uint8)
    blocks = np.zeros((q.shape[0], 66), np.uint8)
    blocks[:, :64] = q.reshape(-1, 64)
    blocks[:, 64] = d_bits & 0xFF
    blocks[:, 65] = d_bits >> 8
    return blocks.reshape(-1)


def encode_tq1_0(trits, d_bits: int = 0x3800) -> np.ndarray:
    """256 trits per block as base-3 fractions (first trit most significant), rounded up: q = ceil(v * 256 / 243);
    32 bytes of 5 digits, 16 bytes of 5 digits, 4 bytes of 4 digits, then the f16 scale."""
    t = np.asarray(trits, np.int64).reshape(-1, 256) + 1
    nb = t.shape[0]
    blocks = np.zeros((nb, 54), np.uint8)

    def ceil(v):
        return (v * 256 + 242) // 243

    a = t[:, :160].reshape(nb, 5, 32)
    blocks[:, :32] = ceil(sum(a[:, n] * 3 ** (4 - n) for n in range(5)))
    b = t[:, 160:240].reshape(nb, 5, 16)
    blocks[:, 32:48] = ceil(sum(b[:, n] * 3 ** (4 - n) for n in range(5)))
    c = t[:, 240:].reshape(nb, 4, 4)
    blocks[:, 48:52] = ceil(sum(c[:, n] * 3 ** (3 - n) for n in range(4)) * 3)
    blocks[:, 52] = d_bits & 0xFF
    blocks[:, 53] = d_bits >> 8
    return blocks.reshape(-1)


def encode_q2_0(trits, scales_f16) -> np.ndarray:
    """Blocks of 64 weights: f16 scale, then 16 bytes of 2-bit codes (code = trit + 1), lowest bits first."""
    t = np.asarray(trits, np.int64).reshape(-1, 16, 4) + 1
    packed = (t[:, :, 0] | (t[:, :, 1] << 2) | (t[:, :, 2] << 4) | (t[:, :, 3] << 6)).astype(np.uint8)
    out = np.zeros((t.shape[0], 18), np.uint8)
    out[:, :2] = np.asarray(scales_f16, np.float16).reshape(-1).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = packed
    return out.reshape(-1)


def _string(s: str) -> bytes:
    raw = s.encode("utf-8")
    return struct.pack("<Q", len(raw)) + raw


def _value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<IB", 7, int(v))
    if isinstance(v, (int, np.integer)):
        return struct.pack("<II", 4, int(v))
    if isinstance(v, (float, np.floating)):
        return struct.pack("<If", 6, float(v))
    if isinstance(v, str):
        return struct.pack("<I", 8) + _string(v)
    if isinstance(v, (list, tuple)) and not v:  # an empty array of strings (a tokenizer without merges)
        return struct.pack("<IIQ", 9, 8, 0)
    if isinstance(v, (list, tuple)):
        bodies = [_value(x) for x in v]
        kinds = {b[:4] for b in bodies}
        if len(kinds) != 1:
            raise TypeError("array items must share one type")
        return struct.pack("<I", 9) + bodies[0][:4] + struct.pack("<Q", len(v)) + b"".join(b[4:] for b in bodies)
    raise TypeError(f"unsupported metadata value {v!r}")


def write_gguf(path, metadata: dict, tensors) -> None:
    """`tensors`: iterable of (name, dims innermost first, ggml type, payload bytes). Payloads start on multiples of 32
    bytes inside the data section; a payload may be longer than the tensor's nominal size (the scale behind I2_S)."""
    tensors = [(name, dims, ggml_type, memoryview(payload).cast("B")) for name, dims, ggml_type, payload in tensors]  # bytes or contiguous arrays
    head = bytearray(b"GGUF") + struct.pack("<IQQ", 3, len(tensors), len(metadata))
    for key, value in metadata.items():
        head += _string(key) + _value(value)
    offsets, cursor = [], 0
    for _, _, _, payload in tensors:
        offsets.append(cursor)
        cursor += (len(payload) + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
    for (name, dims, ggml_type, _), off in zip(tensors, offsets):
        head += _string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", int(d)) for d in dims) + struct.pack("<IQ", ggml_type, off)
    head += b"\0" * (-len(head) % ALIGNMENT)
    with open(path, "wb") as f:
        f.write(head)
        for _, _, _, payload in tensors:
            f.write(payload)
            f.write(b"\0" * (-len(payload) % ALIGNMENT))


def write_model_gguf(path, spec: dict, trits: list, encoding: int = GGML_I2_S, architecture: str = "llama", name: str = "synthetic",
                     extra_metadata: dict | None = None) -> None:
    """Writes the model `spec` (dimensions, scales, norms, embed, lm_head, out_norm as in synth.make_model) with the
    ternary projections `trits` (layers * 7 arrays [rows, cols], order q, k, v, o, gate, up, down) in `encoding`.
    TQ encodings store the tensor scale as the f16 of every block, so the scales must be exactly representable in f16.
    `extra_metadata` is added to the file's key/value pairs (a tokenizer, for instance)."""
    L, H, I, hd = spec["layers"], spec["hidden"], spec["inter"], spec["head_dim"]
    qd, kvd = spec["q_heads"] * hd, spec["kv_heads"] * hd
    shapes = [(qd, H), (kvd, H), (kvd, H), (H, qd), (I, H), (I, H), (H, I)]
    names = ["attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"]
    meta = {
        "general.architecture": architecture, "general.name": name, "general.alignment": ALIGNMENT,
        f"{architecture}.vocab_size": spec["vocab"], f"{architecture}.embedding_length": H, f"{architecture}.feed_forward_length": I,
        f"{architecture}.block_count": L, f"{architecture}.attention.head_count": spec["q_heads"],
        f"{architecture}.attention.head_count_kv": spec["kv_heads"], f"{architecture}.attention.key_length": hd,
        f"{architecture}.attention.layer_norm_rms_epsilon": float(spec["eps"]), f"{architecture}.rope.freq_base": float(spec["rope_theta"]),
        f"{architecture}.rope.dimension_count": spec["rope_dims"], f"{architecture}.context_length": spec["ctx"],
    }
    meta.update(extra_metadata or {})
    table_type = GGML_BF16 if spec.get("bf16_tables") else GGML_F16
    tensors = [("token_embd.weight", (H, spec["vocab"]), table_type, np.ascontiguousarray(spec["embed"], np.uint16).tobytes())]
    norm_names = ["attn_norm", "ffn_norm", "attn_sub_norm", "ffn_sub_norm"]
    for l in range(L):
        for k in range(7):
            rows, cols = shapes[k]
            t = np.asarray(trits[l * 7 + k], np.int8).reshape(rows, cols)
            scale = np.float32(spec["scales"][l * 7 + k])
            if encoding == GGML_Q2_0:  # one f16 scale per 64 weights, from spec["block_scales"] (exact in f16)
                bsc = np.asarray(spec["block_scales"][l * 7 + k], np.float32)
                if not np.array_equal(bsc.astype(np.float16).astype(np.float32), bsc):
                    raise ValueError("Q2_0 needs block scales that are exact in f16")
                payload = encode_q2_0(t, bsc.astype(np.float16)).tobytes()
            elif encoding == GGML_I2_S:
                payload = encode_i2_s(t, rows, cols).tobytes() + struct.pack("<f", float(scale))
            else:
                d_bits = int(np.float16(scale).view(np.uint16))
                if np.float32(np.float16(scale)) != scale:
                    raise ValueError("TQ encodings need scales that are exact in f16")
                payload = (encode_tq1_0(t, d_bits) if encoding == GGML_TQ1_0 else encode_tq2_0(t, d_bits)).tobytes()
            tensors.append((f"blk.{l}.{names[k]}.weight", (cols, rows), encoding, payload))
        for k in range(4):
            w = spec["norms"][l * 4 + k]
            if w is not None:
                tensors.append((f"blk.{l}.{norm_names[k]}.weight", (len(w),), GGML_F32, np.ascontiguousarray(w, np.float32).tobytes()))
        for k, nm in enumerate(("attn_q_norm", "attn_k_norm")):  # query/key head norms (Qwen3), head_dim values each
            if spec.get("qk_norms"):
                tensors.append((f"blk.{l}.{nm}.weight", (hd,), GGML_F32, np.ascontiguousarray(spec["qk_norms"][l * 2 + k], np.float32).tobytes()))
    tensors.append(("output_norm.weight", (H,), GGML_F32, np.ascontiguousarray(spec["out_norm"], np.float32).tobytes()))
    if spec.get("lm_head") is not None:
        tensors.append(("output.weight", (H, spec["vocab"]), table_type, np.ascontiguousarray(spec["lm_head"], np.uint16).tobytes()))
    write_gguf(path, meta, tensors)


# ---- the same encodings on a torch device, and full-size model files -------------------------------------------------

def torch_encode(encoding: int, digits, d_bits: int = 0x3800, block_scales=None):
    """Payload (uint8 tensor on the digits' device) of a [rows, cols] tensor of digits trit + 1 in `encoding`; the same bytes
    as the numpy encoders above. d_bits: the F16 scale every TQ block carries; block_scales: float tensor, one per 64 weights."""
    import torch

    rows, cols = digits.shape
    d = digits.to(torch.int32)
    if encoding == GGML_I2_S:
        t = d.view(rows, cols // 128, 4, 32)
        return ((t[:, :, 0] << 6) | (t[:, :, 1] << 4) | (t[:, :, 2] << 2) | t[:, :, 3]).to(torch.uint8).reshape(-1)
    if encoding == GGML_TQ2_0:
        t = d.view(-1, 2, 4, 32)
        q = (t[:, :, 0] | (t[:, :, 1] << 2) | (t[:, :, 2] << 4) | (t[:, :, 3] << 6)).to(torch.uint8).reshape(-1, 64)
        blocks = torch.empty((q.shape[0], 66), dtype=torch.uint8, device=digits.device)
        blocks[:, :64] = q
        blocks[:, 64], blocks[:, 65] = d_bits & 0xFF, d_bits >> 8
        return blocks.reshape(-1)
    if encoding == GGML_TQ1_0:
        t = d.view(-1, 256)
        nb = t.shape[0]
        blocks = torch.empty((nb, 54), dtype=torch.uint8, device=digits.device)
        a, b, c = t[:, :160].reshape(nb, 5, 32), t[:, 160:240].reshape(nb, 5, 16), t[:, 240:].reshape(nb, 4, 4)
        blocks[:, :32] = ((sum(a[:, n] * 3 ** (4 - n) for n in range(5)) * 256 + 242) // 243).to(torch.uint8)
        blocks[:, 32:48] = ((sum(b[:, n] * 3 ** (4 - n) for n in range(5)) * 256 + 242) // 243).to(torch.uint8)
        blocks[:, 48:52] = ((sum(c[:, n] * 3 ** (3 - n) for n in range(4)) * 3 * 256 + 242) // 243).to(torch.uint8)
        blocks[:, 52], blocks[:, 53] = d_bits & 0xFF, d_bits >> 8
        return blocks.reshape(-1)
    if encoding == GGML_Q2_0:
        t = d.view(-1, 16, 4)
        out = torch.empty((t.shape[0], 18), dtype=torch.uint8, device=digits.device)
        out[:, :2] = block_scales.to(torch.float16).view(torch.uint8).reshape(-1, 2)
        out[:, 2:] = (t[:, :, 0] | (t[:, :, 1] << 2) | (t[:, :, 2] << 4) | (t[:, :, 3] << 6)).to(torch.uint8)
        return out.reshape(-1)
    raise ValueError(f"no encoder for GGML type {encoding}")


def write_full_model_gguf(path, shape: str, encoding: int, device, ctx: int, bf16_tables: bool = False, layers: int | None = None) -> dict:
    """Writes the named full-size model (quintrit_b200.synth.full_model: "falcon3_10b" or "bitnet_2b", every value
    machine-independent) as a GGUF file with its projections in `encoding`, building and encoding every tensor on `device`.
    I2_S files carry float32 tensor scales, TQ1_0 / TQ2_0 files the same scales rounded to F16 in every block, Q2_0 files one
    F16 scale per 64 weights. Returns the model's dimensions."""
    import torch

    from . import synth

    d = synth.full_dims(shape, layers)
    variant = {GGML_I2_S: "i2_s", GGML_TQ1_0: "tq", GGML_TQ2_0: "tq", GGML_Q2_0: "q2_0"}[encoding]
    a, H, L = d["gguf_arch"], d["hidden"], d["layers"]
    meta = {
        "general.architecture": a, "general.name": d["name"], "general.alignment": ALIGNMENT,
        f"{a}.vocab_size": d["vocab"], f"{a}.embedding_length": H, f"{a}.feed_forward_length": d["inter"], f"{a}.block_count": L,
        f"{a}.attention.head_count": d["q_heads"], f"{a}.attention.head_count_kv": d["kv_heads"], f"{a}.attention.key_length": d["head_dim"],
        f"{a}.attention.layer_norm_rms_epsilon": float(d["eps"]), f"{a}.rope.freq_base": float(d["rope_theta"]),
        f"{a}.rope.dimension_count": d["rope_dims"], f"{a}.context_length": ctx,
    }
    config = d["config"]
    table_type = GGML_BF16 if bf16_tables else GGML_F16
    tensors = [("token_embd.weight", (H, d["vocab"]), table_type, synth.torch_table_bits(synth.seed_for(config, 255, 0, 0), d["vocab"] * H, bf16_tables, device).data)]
    names = ["attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"]
    ones = lambda n: np.ones(n, np.float32).data  # noqa: E731
    qd = d["q_heads"] * d["head_dim"]
    for l in range(L):
        for k, (rows, cols) in enumerate(d["shapes"]):
            digits = synth.torch_digits(synth.seed_for(config, l, k, 0), rows, cols, device)
            scale = synth.full_scale(config, l, k, variant)
            if encoding == GGML_Q2_0:
                bsc = torch.from_numpy(synth.torch_block_scales(synth.seed_for(config, l, k, 1), rows * cols // 64, device)).to(device)
                payload = torch_encode(encoding, digits, block_scales=bsc).cpu().numpy().data
            elif encoding == GGML_I2_S:
                payload = memoryview(torch_encode(encoding, digits).cpu().numpy().tobytes() + struct.pack("<f", float(scale)))
            else:
                payload = torch_encode(encoding, digits, d_bits=int(np.float16(scale).view(np.uint16))).cpu().numpy().data
            tensors.append((f"blk.{l}.{names[k]}.weight", (cols, rows), encoding, payload))
        tensors.append((f"blk.{l}.attn_norm.weight", (H,), GGML_F32, ones(H)))
        tensors.append((f"blk.{l}.ffn_norm.weight", (H,), GGML_F32, ones(H)))
        if d["arch"] == 1:
            tensors.append((f"blk.{l}.attn_sub_norm.weight", (qd,), GGML_F32, ones(qd)))
            tensors.append((f"blk.{l}.ffn_sub_norm.weight", (d["inter"],), GGML_F32, ones(d["inter"])))
    tensors.append(("output_norm.weight", (H,), GGML_F32, ones(H)))
    if not d["tied"]:
        tensors.append(("output.weight", (H, d["vocab"]), table_type, synth.torch_table_bits(synth.seed_for(config, 255, 1, 0), d["vocab"] * H, bf16_tables, device).data))
    write_gguf(path, meta, tensors)
    return d
