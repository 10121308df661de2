"""Pre-transcoded model container: a GGUF file whose ternary projections are stored as planar velurex rows (1.60 bits per weight,
the reference's packed format, `rust/crates/quintrit-core/src/pack.rs:28-131`) with their scale, so that loading a model decodes
nothing (the reference's roadmap calls this the `.quintrit` container, `docs/architecture.md:65-72`).

The container is a GGUF file like its source: every metadata entry (tokenizer included) and every dense tensor is copied as it is;
an I2_S / TQ1_0 / TQ2_0 projection becomes a tensor of type `GGML_VELUREX` (not a GGML type; the loaders of this library know it)
whose payload is `rows x ceil(cols / 160) x 32` bytes followed by the tensor's f32 scale. Two metadata entries are added:
`quintrit_b200.container_version` and `quintrit_b200.f32_values` (which attention numerics the source file selected: the reference
decides that by the tensor types it finds, and the container no longer has them). Q2_0 projections stay as they are (their
per-block scales live inside their payload). The transcoding runs on the GPU (`quintrit_gguf_convert_tensor`).
"""
from __future__ import annotations

import struct

import numpy as np

from . import gguf_io

GGML_VELUREX = 0x5156
CONTAINER_VERSION = 1
_TERNARY = {34, 35, 36}  # TQ1_0, TQ2_0, I2_S
_SCALAR = {0: 1, 1: 1, 2: 2, 3: 2, 4: 4, 5: 4, 6: 4, 7: 1, 10: 8, 11: 8, 12: 8}


def _skip_value(buf: memoryview, at: int, kind: int) -> int:
    if kind in _SCALAR:
        return at + _SCALAR[kind]
    if kind == 8:
        (n,) = struct.unpack_from("<Q", buf, at)
        return at + 8 + n
    if kind == 9:
        elem, count = struct.unpack_from("<IQ", buf, at)
        at += 12
        for _ in range(count):
            at = _skip_value(buf, at, elem)
        return at
    raise ValueError(f"metadata value of unknown type {kind}")


def read_directory(raw: bytes):
    """(version, metadata bytes, number of entries, alignment, tensors [(name, dims, type, offset)], start of the data section)."""
    buf = memoryview(raw)
    if bytes(buf[:4]) != b"GGUF":
        raise ValueError("not a GGUF file")
    version, n_tensors, n_kv = struct.unpack_from("<IQQ", buf, 4)
    at = kv0 = 24
    alignment = gguf_io.ALIGNMENT
    for _ in range(n_kv):
        (klen,) = struct.unpack_from("<Q", buf, at)
        key = bytes(buf[at + 8:at + 8 + klen]).decode("utf-8")
        at += 8 + klen
        (kind,) = struct.unpack_from("<I", buf, at)
        if key == "general.alignment" and kind == 4:
            (alignment,) = struct.unpack_from("<I", buf, at + 4)
        at = _skip_value(buf, at + 4, kind)
    kv1 = at
    tensors = []
    for _ in range(n_tensors):
        (nlen,) = struct.unpack_from("<Q", buf, at)
        name = bytes(buf[at + 8:at + 8 + nlen]).decode("utf-8")
        at += 8 + nlen
        (rank,) = struct.unpack_from("<I", buf, at)
        dims = list(struct.unpack_from(f"<{rank}Q", buf, at + 4))
        at += 4 + 8 * rank
        kind, off = struct.unpack_from("<IQ", buf, at)
        at += 12
        tensors.append((name, dims, kind, off))
    data_start = (at + alignment - 1) // alignment * alignment
    return version, bytes(buf[kv0:kv1]), n_kv, alignment, tensors, data_start


def _payload_sizes(tensors, data_start: int, file_size: int):
    """Bytes from every tensor's offset to the next tensor's (or the end of the file): covers a scale stored behind a payload."""
    order = sorted(range(len(tensors)), key=lambda i: tensors[i][3])
    sizes = [0] * len(tensors)
    for k, i in enumerate(order):
        end = tensors[order[k + 1]][3] if k + 1 < len(order) else file_size - data_start
        sizes[i] = end - tensors[i][3]
    return sizes


def convert(src, dst, transcode=None) -> dict:
    """Writes the container of the GGUF model `src` to `dst`. `transcode(name) -> (planar bytes, rows, cols, scale)` defaults to the
    library's on-device transcoder. Returns counts of what was converted."""
    with open(src, "rb") as f:
        raw = f.read()
    version, kv_bytes, n_kv, alignment, tensors, data_start = read_directory(raw)
    if alignment != gguf_io.ALIGNMENT:
        raise ValueError(f"alignment {alignment} is not supported")
    opened = None
    if transcode is None:
        from .runtime import GgufFile

        opened = GgufFile(src)
        transcode = opened.convert_tensor
    sizes = _payload_sizes(tensors, data_start, len(raw))
    out, converted, has_i2s = [], 0, any(kind == 36 for _, _, kind, _ in tensors)
    for (name, dims, kind, off), size in zip(tensors, sizes):
        if kind in _TERNARY and len(dims) == 2:
            planar, rows, cols, scale = transcode(name)
            assert [cols, rows] == dims
            out.append((name, dims, GGML_VELUREX, np.concatenate([np.asarray(planar, np.uint8), np.frombuffer(np.float32(scale).tobytes(), np.uint8)])))
            converted += 1
        else:
            out.append((name, dims, kind, raw[data_start + off:data_start + off + size]))
    if opened is not None:
        opened.close()
    extra = gguf_io._string("quintrit_b200.container_version") + gguf_io._value(CONTAINER_VERSION) + gguf_io._string("quintrit_b200.f32_values") + gguf_io._value(0 if has_i2s else 1)
    head = bytearray(b"GGUF") + struct.pack("<IQQ", version, len(out), n_kv + 2) + kv_bytes + extra
    cursor, offsets = 0, []
    for _, _, _, payload in out:
        offsets.append(cursor)
        cursor += (len(payload) + alignment - 1) // alignment * alignment
    for (name, dims, kind, _), off in zip(out, offsets):
        head += gguf_io._string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", int(d)) for d in dims) + struct.pack("<IQ", kind, off)
    head += b"\0" * (-len(head) % alignment)
    with open(dst, "wb") as f:
        f.write(head)
        for _, _, _, payload in out:
            payload = memoryview(payload).cast("B")
            f.write(payload)
            f.write(b"\0" * (-len(payload) % alignment))
    return {"tensors": len(out), "converted": converted, "source_bytes": len(raw), "container_bytes": len(head) + cursor}
