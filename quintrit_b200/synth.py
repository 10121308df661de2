"""Seeded synthetic inputs for the benchmark configurations (no dataset is involved anywhere).

Generator: counter-based SplitMix64. Value ``i`` of a stream is ``mix(seed + (i + 1) * GAMMA)``; the 32 high bits are
the uniform ``u``. Trits: ``u < 0.3 * 2^32 -> -1``, ``u < 0.6 * 2^32 -> +1``, else ``0`` (P = 0.3 / 0.3 / 0.4).
Weight scale: ``0.5 + 1.5 * u / 2^32`` in fp32. Activations: N(0, 1) by Box-Muller on two uniforms in fp32, then the
int8 absmax quantiser of the caller. Seeds: ``BASE ^ (config << 48) ^ (layer << 16) ^ (projection << 8) ^ stream`` with
projection order q, k, v, o, gate, up, down = 0..6 and streams 0 = weights, 1 = scale, 2 = activation.

The numpy functions are the definition; the torch functions compute the same integers on a CUDA device so that the
9.5 G weights of a Falcon3-10B-shape sweep are generated in seconds (tests/test_synth.py checks they agree).
"""
from __future__ import annotations

import numpy as np

BASE_SEED = 0x5155494E54524954
GAMMA = 0x9E3779B97F4A7C15
M1 = 0xBF58476D1CE4E5B9
M2 = 0x94D049BB133111EB
T_NEG = int(0.3 * 2 ** 32)
T_POS = int(0.6 * 2 ** 32)
PROJECTIONS = ("q", "k", "v", "o", "gate", "up", "down")
# Packer used by make_model: None = the library's own quintrit_b200_pack_planar. The test suite installs the CPU oracle's
# independent packer here, so that the bytes the oracle decodes in decoder tests were not produced by the code under test.
PACKER = None


def falcon3_10b_shapes():
    """(rows N, cols K) of the seven projections of one Falcon3-10B layer, in model order."""
    return [(3072, 3072), (1024, 3072), (1024, 3072), (3072, 3072), (23040, 3072), (23040, 3072), (3072, 23040)]


def bitnet_2b_shapes():
    return [(2560, 2560), (640, 2560), (640, 2560), (2560, 2560), (6912, 2560), (6912, 2560), (2560, 6912)]


def seed_for(config: int, layer: int, projection: int, stream: int) -> int:
    return (BASE_SEED ^ (config << 48) ^ (layer << 16) ^ (projection << 8) ^ stream) & 0xFFFFFFFFFFFFFFFF


def splitmix_u32(seed: int, start: int, n: int) -> np.ndarray:
    """Uniform 32-bit values ``start .. start + n`` of the stream ``seed`` (numpy, the definition)."""
    with np.errstate(over="ignore"):
        i = np.arange(start + 1, start + n + 1, dtype=np.uint64)
        z = np.uint64(seed) + i * np.uint64(GAMMA)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(M1)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(M2)
        z = z ^ (z >> np.uint64(31))
    return (z >> np.uint64(32)).astype(np.uint32)


def trits(seed: int, n: int, start: int = 0) -> np.ndarray:
    u = splitmix_u32(seed, start, n)
    return np.where(u < T_NEG, -1, np.where(u < T_POS, 1, 0)).astype(np.int8)


def weight_scale(seed: int) -> np.float32:
    u = splitmix_u32(seed, 0, 1)[0]
    return np.float32(0.5) + np.float32(1.5) * (np.float32(u) / np.float32(4294967296.0))


def normal_f32(seed: int, n: int) -> np.ndarray:
    """N(0,1) in fp32 by Box-Muller: pairs (u1, u2) -> sqrt(-2 ln u1) cos(2 pi u2), u1 in (0, 1]."""
    u = splitmix_u32(seed, 0, 2 * n).astype(np.float64)
    u1 = ((u[0::2] + 1.0) / 4294967296.0).astype(np.float32)
    u2 = (u[1::2] / 4294967296.0).astype(np.float32)
    r = np.sqrt(np.float32(-2.0) * np.log(u1)).astype(np.float32)
    return (r * np.cos(np.float32(2.0 * np.pi) * u2).astype(np.float32)).astype(np.float32)


# ---- the same integers on a torch device ---------------------------------------------------------------------------

def _s64(v: int) -> int:
    v &= 0xFFFFFFFFFFFFFFFF
    return v - (1 << 64) if v >= (1 << 63) else v


def torch_splitmix_u32(seed: int, start: int, n: int, device):
    import torch

    i = torch.arange(start + 1, start + n + 1, dtype=torch.int64, device=device)
    z = i * _s64(GAMMA) + _s64(seed)
    z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * _s64(M1)
    z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * _s64(M2)
    z = z ^ ((z >> 31) & ((1 << 33) - 1))
    return (z >> 32) & 0xFFFFFFFF  # int64 holding the unsigned 32-bit value


def torch_planar(seed: int, rows: int, cols: int, device, chunk_rows: int = 4096, row0: int = 0):
    """Planar velurex bytes (uint8 tensor, rows * ceil(cols/160) * 32) of rows ``row0 .. row0 + rows`` of the seeded
    ternary matrix, built on `device`."""
    import torch

    blocks = -(-cols // 160)
    out = torch.empty((rows, blocks * 32), dtype=torch.uint8, device=device)
    radix = torch.tensor([1, 3, 9, 28, 84], dtype=torch.int64, device=device).view(1, 1, 5, 1)
    for r0 in range(0, rows, chunk_rows):
        nr = min(chunk_rows, rows - r0)
        u = torch_splitmix_u32(seed, (row0 + r0) * cols, nr * cols, device).view(nr, cols)
        d = torch.where(u < T_NEG, 0, torch.where(u < T_POS, 2, 1))
        if blocks * 160 != cols:
            d = torch.nn.functional.pad(d, (0, blocks * 160 - cols), value=1)
        out[r0:r0 + nr] = (d.view(nr, blocks, 5, 32) * radix).sum(dim=2).to(torch.uint8).view(nr, blocks * 32)
    return out.view(-1)


def quantize_int8_np(x: np.ndarray):
    """Per-token absmax int8 quantisation of the synthetic activations (s = 127 / max|x|, round half away from zero,
    clamp to [-128, 127]); returns (codes, s). Input preparation for the benchmark, not a product kernel."""
    x = np.asarray(x, np.float32)
    amax = np.float32(np.abs(x).max()) if x.size else np.float32(0)
    if not amax > 0:
        return np.zeros(x.size, np.int8), np.float32(0)
    s = np.float32(127.0) / amax
    y = x * s
    q = np.sign(y) * np.floor(np.abs(y) + np.float32(0.5))
    return np.clip(q, -128, 127).astype(np.int8), s


def make_model(arch: int, f32_values: bool, hidden: int, inter: int, layers: int, q_heads: int, kv_heads: int, head_dim: int, vocab: int,
               ctx: int, rope_theta: float, eps: float, config: int = 1, tied: bool = False, rope_dims: int | None = None,
               random_norms: bool = False, bf16_tables: bool = False) -> dict:
    """A seeded random-init model of the given shape as numpy arrays (planar velurex projections, F16 tables).

    Ternary projections and their scales come from the streams documented at the top of this module; embedding and
    output head are N(0, 0.02) rounded to F16; norm weights are 1.0 (or U(0.5, 1.5) with ``random_norms``, which
    exercises the weight multiply in tests). ``arch`` 1 (BitNet) gets attention and FFN sub-norm weights.
    """
    from . import api

    qd, kvd = q_heads * head_dim, kv_heads * head_dim
    shapes = [(qd, hidden), (kvd, hidden), (kvd, hidden), (hidden, qd), (inter, hidden), (inter, hidden), (hidden, inter)]
    weights, scales, norms = [], [], []

    def norm(seed, n):
        if not random_norms:
            return np.ones(n, np.float32)
        return (np.float32(0.5) + splitmix_u32(seed, 0, n).astype(np.float32) / np.float32(4294967296.0)).astype(np.float32)

    for l in range(layers):
        for p, (rows, cols) in enumerate(shapes):
            weights.append((PACKER or api.pack_planar)(trits(seed_for(config, l, p, 0), rows * cols), rows, cols))
            scales.append(weight_scale(seed_for(config, l, p, 1)))
        norms += [norm(seed_for(config, l, 7, 0), hidden), norm(seed_for(config, l, 7, 1), hidden),
                  norm(seed_for(config, l, 7, 2), qd) if arch == 1 else None, norm(seed_for(config, l, 7, 3), inter) if arch == 1 else None]
    def table(seed):  # N(0, 0.02) as F16 bits, or as BF16 bits rounded to nearest even
        x = normal_f32(seed, vocab * hidden) * np.float32(0.02)
        if not bf16_tables:
            return x.astype(np.float16).view(np.uint16)
        u = x.view(np.uint32)
        return ((u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)).astype(np.uint16)

    embed = table(seed_for(config, 255, 0, 0))
    head = None if tied else table(seed_for(config, 255, 1, 0))
    return dict(bf16_tables=bf16_tables, arch=arch, f32_values=f32_values, hidden=hidden, inter=inter, layers=layers, q_heads=q_heads, kv_heads=kv_heads,
                head_dim=head_dim, vocab=vocab, ctx=ctx, rope_dims=rope_dims or head_dim, eps=eps, rope_theta=rope_theta, weights=weights,
                scales=np.array(scales, np.float32), norms=norms, embed=embed, lm_head=head, out_norm=norm(seed_for(config, 255, 2, 0), hidden))


def torch_normal_f16_bits(seed: int, n: int, std: float, device, chunk: int = 1 << 24) -> np.ndarray:
    """N(0, std) values as F16 bit patterns (numpy uint16), generated on `device` from the seeded stream by Box-Muller."""
    import torch

    out = np.empty(n, np.uint16)
    for s0 in range(0, n, chunk):
        m = min(chunk, n - s0)
        u = torch_splitmix_u32(seed, 2 * s0, 2 * m, device).to(torch.float64)
        u1 = ((u[0::2] + 1.0) / 4294967296.0).to(torch.float32)
        u2 = (u[1::2] / 4294967296.0).to(torch.float32)
        x = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(6.283185307179586 * u2) * std
        out[s0:s0 + m] = x.to(torch.float16).view(torch.int16).cpu().numpy().view(np.uint16)
    return out


def torch_model(shape: str, device, ctx: int, f32_values: bool = False, config: int = 2, layers: int | None = None, tp=None) -> dict:
    """The Falcon3-10B-shape or BitNet-2B-shape model with seeded random-init weights, built on a torch device."""
    if shape == "falcon3_10b":
        arch, hidden, inter, L, qh, kvh, hd, vocab, theta, eps, tied = 0, 3072, 23040, 40, 12, 4, 256, 131072, 1000042.0, 1e-6, False
    elif shape == "bitnet_2b":
        arch, hidden, inter, L, qh, kvh, hd, vocab, theta, eps, tied = 1, 2560, 6912, 30, 20, 5, 128, 128256, 500000.0, 1e-5, True
    else:
        raise ValueError(shape)
    L = layers or L
    qd, kvd = qh * hd, kvh * hd
    shapes = [(qd, hidden), (kvd, hidden), (kvd, hidden), (hidden, qd), (inter, hidden), (inter, hidden), (hidden, inter)]
    weights, scales, norms = [], [], []
    for l in range(L):
        for p, (rows, cols) in enumerate(shapes):
            if tp is None:
                w = torch_planar(seed_for(config, l, p, 0), rows, cols, device)
            elif p < 3 and kvh % tp[1] != 0:  # the ranks do not divide the KV heads: q, k and v whole on every rank (see shard_spec)
                w = torch_planar(seed_for(config, l, p, 0), rows, cols, device)
            else:  # only this rank's rows
                n = rows // tp[1]
                w = torch_planar(seed_for(config, l, p, 0), n, cols, device, row0=tp[0] * n)
            weights.append(w.cpu().numpy().reshape(-1))
            scales.append(weight_scale(seed_for(config, l, p, 1)))
        norms += [np.ones(hidden, np.float32), np.ones(hidden, np.float32), np.ones(qd, np.float32) if arch == 1 else None,
                  np.ones(inter, np.float32) if arch == 1 else None]
    embed = torch_normal_f16_bits(seed_for(config, 255, 0, 0), vocab * hidden, 0.02, device)
    head = None if tied else torch_normal_f16_bits(seed_for(config, 255, 1, 0), vocab * hidden, 0.02, device)
    spec = dict(arch=arch, f32_values=f32_values, hidden=hidden, inter=inter, layers=L, q_heads=qh, kv_heads=kvh, head_dim=hd, vocab=vocab,
                ctx=ctx, rope_dims=hd, eps=eps, rope_theta=theta, weights=weights, scales=np.array(scales, np.float32), norms=norms,
                embed=embed, lm_head=head, out_norm=np.ones(hidden, np.float32), shape=shape)
    if tp is not None:
        spec.update(tp_rank=tp[0], tp_world=tp[1])
        if head is not None:
            v = vocab // tp[1]
            spec["lm_head"] = np.ascontiguousarray(head.reshape(vocab, hidden)[tp[0] * v:(tp[0] + 1) * v]).reshape(-1)
    return spec


def prompt_tokens(config: int, n: int, vocab: int) -> np.ndarray:
    """Uniform token ids from stream 3."""
    return (splitmix_u32(seed_for(config, 0, 0, 3), 0, n).astype(np.uint64) * np.uint64(vocab) >> np.uint64(32)).astype(np.uint32)


def batch_lengths(config: int, n: int, lo: int = 256, hi: int = 2048) -> np.ndarray:
    """Prompt lengths of a batch of sequences, uniform in [lo, hi], from stream 4."""
    u = splitmix_u32(seed_for(config, 0, 0, 4), 0, n).astype(np.uint64)
    return (np.uint64(lo) + (u * np.uint64(hi - lo + 1) >> np.uint64(32))).astype(np.int64)


def shard_spec(spec: dict, rank: int, world: int) -> dict:
    """The share of `spec` (planar numpy projections) that rank `rank` of a tensor-parallel group of `world` GPUs holds:
    its rows of every projection - q / k / v rows of its heads, rows [rank * n / world, (rank + 1) * n / world) of o,
    gate, up and down - and its rows of the output head. Dimensions stay those of the whole model. Where `world` does not
    divide the KV heads, q, k and v stay whole on every rank (attention is replicated, the rest is split)."""
    from . import api

    H, I, hd = spec["hidden"], spec["inter"], spec["head_dim"]
    qd, kvd = spec["q_heads"] * hd, spec["kv_heads"] * hd
    assert H % world == 0 and I % world == 0 and spec["vocab"] % world == 0
    replicated = spec["kv_heads"] % world != 0
    shapes = [(qd, H), (kvd, H), (kvd, H), (H, qd), (I, H), (I, H), (H, I)]
    weights = []
    for i, w in enumerate(spec["weights"]):
        rows, cols = shapes[i % 7]
        rb = api.row_bytes(cols)
        if replicated and i % 7 < 3:
            weights.append(np.ascontiguousarray(np.asarray(w, np.uint8)).reshape(-1))
            continue
        n = rows // world
        weights.append(np.ascontiguousarray(np.asarray(w, np.uint8).reshape(rows, rb)[rank * n:(rank + 1) * n]).reshape(-1))
    out = dict(spec, weights=weights, tp_rank=rank, tp_world=world)
    if spec.get("lm_head") is not None:
        v = spec["vocab"] // world
        out["lm_head"] = np.ascontiguousarray(np.asarray(spec["lm_head"], np.uint16).reshape(spec["vocab"], H)[rank * v:(rank + 1) * v]).reshape(-1)
    return out


# ---- full-size models whose every value is the same on any machine --------------------------------------------------
# The sequences of the full-size parity fixtures are computed on one machine (CPU) and checked on another (GPU box), so
# nothing in these models may depend on a libm or on a device's float kernels: trits and scales come from integer
# arithmetic and single IEEE operations, and the dense tables replace Box-Muller by a sum of four uniforms.

TABLE_STD = 0.02
_TABLE_GAIN = TABLE_STD * 1.7320508075688772 / 4294967296.0  # sum of four U[0, 2^32): mean 2^33, standard deviation 2^32 / sqrt(3)


def _bits_from_f32(x, bf16: bool):
    """F16 or BF16 (round to nearest even) bit patterns of a float32 numpy array."""
    if not bf16:
        return x.astype(np.float16).view(np.uint16)
    u = x.view(np.uint32)
    return ((u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)).astype(np.uint16)


def table_bits_np(seed: int, n: int, bf16: bool = False, start: int = 0) -> np.ndarray:
    """Values ``start .. start + n`` of a dense table: (u0 + u1 + u2 + u3 - 2^33) * gain with four consecutive uniforms
    of the stream, one float64 multiply (exact inputs), rounded to float32 and then to F16 / BF16. Bell-shaped with
    standard deviation 0.02; identical on every IEEE machine (numpy definition)."""
    u = splitmix_u32(seed, 4 * start, 4 * n).astype(np.int64).reshape(n, 4).sum(axis=1)
    x = ((u - (1 << 33)).astype(np.float64) * _TABLE_GAIN).astype(np.float32)
    return _bits_from_f32(x, bf16)


def torch_table_bits(seed: int, n: int, bf16: bool, device, chunk: int = 1 << 23) -> np.ndarray:
    """table_bits_np computed on a torch device (same integers, same single multiply)."""
    import torch

    out = np.empty(n, np.uint16)
    for s0 in range(0, n, chunk):
        m = min(chunk, n - s0)
        u = torch_splitmix_u32(seed, 4 * s0, 4 * m, device).view(m, 4).sum(dim=1)
        x = ((u - (1 << 33)).to(torch.float64) * _TABLE_GAIN).to(torch.float32)
        h = x.to(torch.bfloat16 if bf16 else torch.float16).view(torch.int16)
        out[s0:s0 + m] = h.cpu().numpy().view(np.uint16)
    return out


def block_scales_np(seed: int, n: int, start: int = 0) -> np.ndarray:
    """Q2_0 block scales: 0.5 + 1.5 u / 2^32 (exact in float64), rounded to float32 and to F16; returned as float32."""
    u = splitmix_u32(seed, start, n).astype(np.float64)
    return (0.5 + 1.5 * u / 4294967296.0).astype(np.float32).astype(np.float16).astype(np.float32)


def torch_block_scales(seed: int, n: int, device, chunk: int = 1 << 24) -> np.ndarray:
    import torch

    out = np.empty(n, np.float32)
    for s0 in range(0, n, chunk):
        m = min(chunk, n - s0)
        u = torch_splitmix_u32(seed, s0, m, device).to(torch.float64)
        out[s0:s0 + m] = (0.5 + 1.5 * u / 4294967296.0).to(torch.float32).to(torch.float16).to(torch.float32).cpu().numpy()
    return out


def torch_digits(seed: int, rows: int, cols: int, device, row0: int = 0):
    """Digits trit + 1 (uint8 tensor [rows, cols]) of the seeded ternary matrix."""
    import torch

    u = torch_splitmix_u32(seed, row0 * cols, rows * cols, device).view(rows, cols)
    return torch.where(u < T_NEG, 0, torch.where(u < T_POS, 2, 1)).to(torch.uint8)


FULL_SHAPES = {
    # arch, hidden, inter, layers, q heads, kv heads, head_dim, vocab, rope theta, eps, tied head, seed field, GGUF architecture, name
    "falcon3_10b": (0, 3072, 23040, 40, 12, 4, 256, 131072, 1000042.0, 1e-6, False, 2, "llama", "falcon3-10b-shape"),
    "bitnet_2b": (1, 2560, 6912, 30, 20, 5, 128, 128256, 500000.0, 1e-5, True, 1, "bitnet-b1.58", "bitnet-2b-shape"),
}


def full_dims(shape: str, layers: int | None = None) -> dict:
    arch, hidden, inter, L, qh, kvh, hd, vocab, theta, eps, tied, config, gguf_arch, name = FULL_SHAPES[shape]
    L = layers or L
    qd, kvd = qh * hd, kvh * hd
    return dict(arch=arch, hidden=hidden, inter=inter, layers=L, q_heads=qh, kv_heads=kvh, head_dim=hd, vocab=vocab, rope_theta=theta, eps=eps,
                tied=tied, config=config, gguf_arch=gguf_arch, name=name, rope_dims=hd,
                shapes=[(qd, hidden), (kvd, hidden), (kvd, hidden), (hidden, qd), (inter, hidden), (inter, hidden), (hidden, inter)])


def full_scale(config: int, layer: int, projection: int, variant: str) -> np.float32:
    """Tensor scale of a projection: U(0.5, 2) in float32; the TQ encodings store it as the F16 of every block, so their
    variant rounds it to F16 (a Q2_0 model has block scales instead and ignores it)."""
    s = weight_scale(seed_for(config, layer, projection, 1))
    return np.float32(np.float16(s)) if variant == "tq" else s


def full_model(shape: str, variant: str, device, ctx: int, bf16_tables: bool = False, layers: int | None = None) -> dict:
    """The named full-size model as numpy arrays for a decoder description (planar velurex projections), every value
    machine-independent. variant: "i2_s" (float32 tensor scales, FP16-accumulator attention), "tq" (F16-exact tensor
    scales, FP32 accumulators) or "q2_0" (one F16 scale per 64 weights, FP32 accumulators)."""
    d = full_dims(shape, layers)
    config, H = d["config"], d["hidden"]
    weights, scales, norms, block_scales = [], [], [], []
    for l in range(d["layers"]):
        for p, (rows, cols) in enumerate(d["shapes"]):
            weights.append(torch_planar(seed_for(config, l, p, 0), rows, cols, device).cpu().numpy().reshape(-1))
            scales.append(full_scale(config, l, p, variant))
            if variant == "q2_0":
                block_scales.append(torch_block_scales(seed_for(config, l, p, 1), rows * cols // 64, device))
        qd = d["q_heads"] * d["head_dim"]
        norms += [np.ones(H, np.float32), np.ones(H, np.float32), np.ones(qd, np.float32) if d["arch"] == 1 else None,
                  np.ones(d["inter"], np.float32) if d["arch"] == 1 else None]
    embed = torch_table_bits(seed_for(config, 255, 0, 0), d["vocab"] * H, bf16_tables, device)
    head = None if d["tied"] else torch_table_bits(seed_for(config, 255, 1, 0), d["vocab"] * H, bf16_tables, device)
    spec = dict(arch=d["arch"], f32_values=variant != "i2_s", hidden=H, inter=d["inter"], layers=d["layers"], q_heads=d["q_heads"], kv_heads=d["kv_heads"],
                head_dim=d["head_dim"], vocab=d["vocab"], ctx=ctx, rope_dims=d["rope_dims"], eps=d["eps"], rope_theta=d["rope_theta"], weights=weights,
                scales=np.array(scales, np.float32), norms=norms, embed=embed, lm_head=head, out_norm=np.ones(H, np.float32), shape=shape,
                bf16_tables=bf16_tables)
    if variant == "q2_0":
        spec["block_scales"] = block_scales
    return spec
