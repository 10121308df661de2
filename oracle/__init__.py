"""ctypes bindings of the CPU oracle (``oracle/qt_oracle.c``, ``oracle/cpu_gemv.c``).

TEST INFRASTRUCTURE ONLY. The package ``quintrit_b200`` never imports this module; only ``tests/``, the smoke check and
the CPU-baseline leg of ``bench.py`` do, and only to check or to time the CPU restatement of the reference algorithm.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libqt_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compiles the oracle with ``make`` (gcc, a few seconds) and returns the path of the shared object."""
    def stale() -> bool:
        return not os.path.exists(_LIB_PATH) or any(
            os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_LIB_PATH) for f in os.listdir(_HERE) if f.endswith((".c", ".h")))

    if force or stale():
        import fcntl

        with open(os.path.join(_HERE, ".build.lock"), "w") as lock:  # several ranks may get here at once: one of them runs make
            fcntl.flock(lock, fcntl.LOCK_EX)
            try:
                if force or stale():
                    subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True, capture_output=True)
            finally:
                fcntl.flock(lock, fcntl.LOCK_UN)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _declare(_lib)
    return _lib


_u8p, _i8p, _i32p, _i64p, _f32p = (C.POINTER(t) for t in (C.c_uint8, C.c_int8, C.c_int32, C.c_int64, C.c_float))
_sz = C.c_size_t


def _declare(l: C.CDLL) -> None:
    l.qto_pack_5trits.restype = C.c_uint8
    l.qto_pack_5trits.argtypes = [_i8p]
    l.qto_byte_to_trits.argtypes = [C.c_uint8, _i8p]
    for name in ("qto_planar_row_bytes", "qto_tile_row_bytes"):
        getattr(l, name).restype = _sz
        getattr(l, name).argtypes = [_sz]
    l.qto_column_activation_index.restype = _sz
    l.qto_column_activation_index.argtypes = [_sz, _sz, _sz]
    l.qto_pack_planar.argtypes = [_i8p, _sz, _sz, _u8p]
    l.qto_unpack_planar.argtypes = [_u8p, _sz, _sz, _i8p]
    l.qto_tile32.argtypes = [_u8p, _sz, _sz, _u8p]
    l.qto_gemv_bruteforce.argtypes = [_i8p, _sz, _sz, _i8p, _i64p]
    l.qto_gemv_planar.argtypes = [_u8p, _sz, _sz, _i8p, _i32p]
    l.qto_gemv_lut_wide.argtypes = [_u8p, _sz, _sz, _i8p, _i32p]
    l.qto_rescale.argtypes = [_i32p, _sz, C.c_float, C.c_float, _f32p]
    l.qto_quantize_int8.restype = C.c_float
    l.qto_quantize_int8.argtypes = [_f32p, _sz, _i8p]
    for name in ("qto_decode_i2_s", "qto_decode_tq2_0", "qto_decode_tq1_0"):
        getattr(l, name).restype = C.c_int
        getattr(l, name).argtypes = [_u8p, _sz, _sz, _sz, _i8p]
    l.qto_encode_i2_s.restype = C.c_int
    l.qto_encode_i2_s.argtypes = [_i8p, _sz, _sz, _u8p]
    l.qto_decode_q2_0.restype = C.c_long
    l.qto_decode_q2_0.argtypes = [_u8p, _sz, _sz, _sz, _i8p, _f32p]
    l.qto_uniform_block_scale.restype = C.c_int
    l.qto_uniform_block_scale.argtypes = [C.c_int, _u8p, _sz, _f32p]
    l.qto_half_to_f32.restype = C.c_float
    l.qto_half_to_f32.argtypes = [C.c_uint16]
    l.qto_cpu_has_avx512_vbmi.restype = C.c_int
    l.qto_tile64_bytes.restype = _sz
    l.qto_tile64_bytes.argtypes = [_sz, _sz]
    l.qto_tile64.argtypes = [_u8p, _sz, _sz, _u8p]
    l.qto_cpu_gemv_avx512.restype = C.c_int
    l.qto_cpu_gemv_avx512.argtypes = [_u8p, _sz, _sz, _i8p, _i32p, C.c_int]
    l.qto_cpu_gemv_portable.argtypes = [_u8p, _sz, _sz, _i8p, _i32p, C.c_int]
    l.qto_synth_planar.argtypes = [C.c_uint64, _sz, _sz, _sz, _u8p]
    l.qto_synth_table.argtypes = [C.c_uint64, _sz, _sz, C.c_int, C.POINTER(C.c_uint16)]
    l.qto_synth_block_scales.argtypes = [C.c_uint64, _sz, _sz, _f32p]
    l.qto_stream_read_gbs.restype = C.c_double
    l.qto_stream_read_gbs.argtypes = [_u8p, _sz, C.c_int, C.c_int, C.POINTER(C.c_uint64)]


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ---- packing -------------------------------------------------------------------------------------------------------

def pack_5trits(t) -> int:
    a = _c(t, np.int8)
    assert a.size == 5
    return int(lib().qto_pack_5trits(_p(a, _i8p)))


def byte_to_trits(b: int) -> np.ndarray:
    out = np.zeros(5, np.int8)
    lib().qto_byte_to_trits(b, _p(out, _i8p))
    return out


def planar_row_bytes(cols: int) -> int:
    return int(lib().qto_planar_row_bytes(cols))


def tile_row_bytes(cols: int) -> int:
    return int(lib().qto_tile_row_bytes(cols))


def column_activation_index(cols: int, c: int, p: int) -> int:
    return int(lib().qto_column_activation_index(cols, c, p))


def pack_planar(trits, rows: int, cols: int) -> np.ndarray:
    t = _c(trits, np.int8).reshape(-1)
    assert t.size == rows * cols
    out = np.zeros(rows * planar_row_bytes(cols), np.uint8)
    lib().qto_pack_planar(_p(t, _i8p), rows, cols, _p(out, _u8p))
    return out


def unpack_planar(packed, rows: int, cols: int) -> np.ndarray:
    p = _c(packed, np.uint8).reshape(-1)
    assert p.size >= rows * planar_row_bytes(cols)
    out = np.zeros(rows * cols, np.int8)
    lib().qto_unpack_planar(_p(p, _u8p), rows, cols, _p(out, _i8p))
    return out.reshape(rows, cols)


def tile32(planar, rows: int, cols: int) -> np.ndarray:
    assert rows % 32 == 0
    p = _c(planar, np.uint8).reshape(-1)
    out = np.zeros(rows * tile_row_bytes(cols), np.uint8)
    lib().qto_tile32(_p(p, _u8p), rows, cols, _p(out, _u8p))
    return out


def synth_planar(seed: int, rows: int, cols: int, row0: int = 0) -> np.ndarray:
    """Planar bytes of rows [row0, row0 + rows) of the seeded synthetic matrix (quintrit_b200.synth.trits + pack), threaded."""
    out = np.zeros(rows * planar_row_bytes(cols), np.uint8)
    lib().qto_synth_planar(seed & 0xFFFFFFFFFFFFFFFF, rows, cols, row0, _p(out, _u8p))
    return out


def synth_table(seed: int, n: int, bf16: bool = False, start: int = 0) -> np.ndarray:
    """quintrit_b200.synth.table_bits_np, threaded."""
    out = np.zeros(n, np.uint16)
    lib().qto_synth_table(seed & 0xFFFFFFFFFFFFFFFF, n, start, int(bf16), out.ctypes.data_as(C.POINTER(C.c_uint16)))
    return out


def synth_block_scales(seed: int, n: int, start: int = 0) -> np.ndarray:
    """quintrit_b200.synth.block_scales_np, threaded."""
    out = np.zeros(n, np.float32)
    lib().qto_synth_block_scales(seed & 0xFFFFFFFFFFFFFFFF, n, start, _p(out, _f32p))
    return out


def stream_read_gbs(nbytes: int = 1 << 30, threads: int = 0, reps: int = 21) -> float:
    """Read-only streaming rate of the host cores over a buffer of `nbytes` (GB/s, best of `reps`)."""
    buf = np.ones(nbytes, np.uint8)
    sink = C.c_uint64(0)
    return float(lib().qto_stream_read_gbs(_p(buf, _u8p), buf.size, threads or (os.cpu_count() or 1), reps, C.byref(sink)))


def full_model(shape: str, variant: str, ctx: int, bf16_tables: bool = False, layers: int | None = None) -> dict:
    """quintrit_b200.synth.full_model built by the threaded generators of this library (the same values: tests/test_synth.py)."""
    from quintrit_b200 import synth

    d = synth.full_dims(shape, layers)
    config, H = d["config"], d["hidden"]
    weights, scales, norms, block_scales = [], [], [], []
    for l in range(d["layers"]):
        for p, (rows, cols) in enumerate(d["shapes"]):
            weights.append(synth_planar(synth.seed_for(config, l, p, 0), rows, cols))
            scales.append(synth.full_scale(config, l, p, variant))
            if variant == "q2_0":
                block_scales.append(synth_block_scales(synth.seed_for(config, l, p, 1), rows * cols // 64))
        qd = d["q_heads"] * d["head_dim"]
        norms += [np.ones(H, np.float32), np.ones(H, np.float32), np.ones(qd, np.float32) if d["arch"] == 1 else None,
                  np.ones(d["inter"], np.float32) if d["arch"] == 1 else None]
    embed = synth_table(synth.seed_for(config, 255, 0, 0), d["vocab"] * H, bf16_tables)
    head = None if d["tied"] else synth_table(synth.seed_for(config, 255, 1, 0), d["vocab"] * H, bf16_tables)
    spec = dict(arch=d["arch"], f32_values=variant != "i2_s", hidden=H, inter=d["inter"], layers=d["layers"], q_heads=d["q_heads"], kv_heads=d["kv_heads"],
                head_dim=d["head_dim"], vocab=d["vocab"], ctx=ctx, rope_dims=d["rope_dims"], eps=d["eps"], rope_theta=d["rope_theta"], weights=weights,
                scales=np.array(scales, np.float32), norms=norms, embed=embed, lm_head=head, out_norm=np.ones(H, np.float32), shape=shape,
                bf16_tables=bf16_tables)
    if variant == "q2_0":
        spec["block_scales"] = block_scales
    return spec


# ---- GEMV ----------------------------------------------------------------------------------------------------------

def gemv_bruteforce(trits, rows: int, cols: int, act) -> np.ndarray:
    t = _c(trits, np.int8).reshape(-1)
    a = _c(act, np.int8)
    assert t.size == rows * cols and a.size == cols
    out = np.zeros(rows, np.int64)
    lib().qto_gemv_bruteforce(_p(t, _i8p), rows, cols, _p(a, _i8p), _p(out, _i64p))
    return out


def gemv_planar(planar, rows: int, cols: int, act) -> np.ndarray:
    p = _c(planar, np.uint8).reshape(-1)
    a = _c(act, np.int8)
    assert p.size >= rows * planar_row_bytes(cols) and a.size == cols
    out = np.zeros(rows, np.int32)
    lib().qto_gemv_planar(_p(p, _u8p), rows, cols, _p(a, _i8p), _p(out, _i32p))
    return out


def gemv_lut_wide(tiled, rows: int, cols: int, act) -> np.ndarray:
    t = _c(tiled, np.uint8).reshape(-1)
    a = _c(act, np.int8)
    assert rows % 32 == 0 and t.size >= rows * tile_row_bytes(cols) and a.size == cols
    out = np.zeros(rows, np.int32)
    lib().qto_gemv_lut_wide(_p(t, _u8p), rows, cols, _p(a, _i8p), _p(out, _i32p))
    return out


def rescale(acc, weight_scale: float, act_scale: float) -> np.ndarray:
    a = _c(acc, np.int32)
    out = np.zeros(a.size, np.float32)
    lib().qto_rescale(_p(a, _i32p), a.size, weight_scale, act_scale, _p(out, _f32p))
    return out


def quantize_int8(x):
    xx = _c(x, np.float32)
    out = np.zeros(xx.size, np.int8)
    s = lib().qto_quantize_int8(_p(xx, _f32p), xx.size, _p(out, _i8p))
    return out, np.float32(s)


# ---- decoders ------------------------------------------------------------------------------------------------------

def _decode(fn, data, rows, cols):
    d = _c(data, np.uint8).reshape(-1)
    out = np.zeros(rows * cols, np.int8)
    rc = fn(_p(d, _u8p), d.size, rows, cols, _p(out, _i8p))
    if rc != 0:
        raise ValueError("payload does not fit the shape")
    return out.reshape(rows, cols)


def decode_i2_s(data, rows, cols):
    return _decode(lib().qto_decode_i2_s, data, rows, cols)


def decode_tq2_0(data, rows, cols):
    return _decode(lib().qto_decode_tq2_0, data, rows, cols)


def decode_tq1_0(data, rows, cols):
    return _decode(lib().qto_decode_tq1_0, data, rows, cols)


def encode_i2_s(trits, rows, cols):
    t = _c(trits, np.int8).reshape(-1)
    out = np.zeros(rows * cols // 4, np.uint8)
    if lib().qto_encode_i2_s(_p(t, _i8p), rows, cols, _p(out, _u8p)) != 0:
        raise ValueError("cols must be a multiple of 128")
    return out


def decode_q2_0(data, rows, cols):
    d = _c(data, np.uint8).reshape(-1)
    trits = np.zeros(rows * cols, np.int8)
    scales = np.zeros(max(rows * cols // 64, 1), np.float32)
    rc = lib().qto_decode_q2_0(_p(d, _u8p), d.size, rows, cols, _p(trits, _i8p), _p(scales, _f32p))
    if rc == -1 and (cols == 0 or cols % 64 != 0 or d.size != rows * cols // 64 * 18):
        raise ValueError("payload does not fit the shape")
    if rc < 0:
        raise ValueError(f"Q2_0 weight {-rc - 1} uses code 3")
    return trits.reshape(rows, cols), scales[: rows * cols // 64]


def uniform_block_scale(ggml_type: int, data):
    d = _c(data, np.uint8).reshape(-1)
    s = C.c_float(0)
    ok = lib().qto_uniform_block_scale(ggml_type, _p(d, _u8p), d.size, C.byref(s))
    return np.float32(s.value) if ok else None


def half_to_f32(h: int) -> np.float32:
    return np.float32(lib().qto_half_to_f32(h))


# ---- timed CPU baseline ---------------------------------------------------------------------------------------------

def cpu_has_avx512_vbmi() -> bool:
    return bool(lib().qto_cpu_has_avx512_vbmi())


def tile64(planar, rows: int, cols: int) -> np.ndarray:
    p = _c(planar, np.uint8).reshape(-1)
    out = np.zeros(lib().qto_tile64_bytes(rows, cols), np.uint8)
    lib().qto_tile64(_p(p, _u8p), rows, cols, _p(out, _u8p))
    return out


def cpu_gemv_avx512(tiled64, rows: int, cols: int, act, threads: int, out=None) -> np.ndarray:
    t = tiled64 if isinstance(tiled64, np.ndarray) and tiled64.dtype == np.uint8 and tiled64.flags.c_contiguous else _c(tiled64, np.uint8)
    a = _c(act, np.int8)
    if out is None:
        out = np.zeros(rows, np.int32)
    if lib().qto_cpu_gemv_avx512(_p(t, _u8p), rows, cols, _p(a, _i8p), _p(out, _i32p), threads) != 0:
        raise RuntimeError("this CPU has no AVX-512 VBMI")
    return out


def cpu_gemv_portable(planar, rows: int, cols: int, act, threads: int, out=None) -> np.ndarray:
    p = planar if isinstance(planar, np.ndarray) and planar.dtype == np.uint8 and planar.flags.c_contiguous else _c(planar, np.uint8)
    a = _c(act, np.int8)
    if out is None:
        out = np.zeros(rows, np.int32)
    lib().qto_cpu_gemv_portable(_p(p, _u8p), rows, cols, _p(a, _i8p), _p(out, _i32p), threads)
    return out


# ---- float decode primitives and the whole-token forward (oracle/qt_oracle_model.c) ---------------------------------

_u16p, _u64p = C.POINTER(C.c_uint16), C.POINTER(C.c_uint64)


def _declare_model(l: C.CDLL) -> None:
    l.qto_f16_to_f32.restype = C.c_float
    l.qto_f16_to_f32.argtypes = [C.c_uint16]
    l.qto_f32_to_f16.restype = C.c_uint16
    l.qto_f32_to_f16.argtypes = [C.c_float]
    l.qto_f32_to_bf16.restype = C.c_uint16
    l.qto_f32_to_bf16.argtypes = [C.c_float]
    l.qto_bf16_to_f32.restype = C.c_float
    l.qto_bf16_to_f32.argtypes = [C.c_uint16]
    l.qto_rms_norm.argtypes = [_f32p, _f32p, _sz, C.c_float, _f32p]
    l.qto_rope_cache.argtypes = [_sz, _sz, C.c_float, _f32p]
    l.qto_rope_apply.argtypes = [_f32p, _sz, _sz, C.c_int, _f32p, _sz]
    l.qto_vec_dot_f16.restype = C.c_float
    l.qto_vec_dot_f16.argtypes = [_u16p, _u16p, _sz]
    l.qto_vec_dot_f16_f32.restype = C.c_float
    l.qto_vec_dot_f16_f32.argtypes = [_u16p, _f32p, _sz]
    l.qto_ggml_expf_lane.restype = C.c_float
    l.qto_ggml_expf_lane.argtypes = [C.c_float]
    l.qto_silu.restype = C.c_float
    l.qto_silu.argtypes = [C.c_float]
    l.qto_swiglu.argtypes = [_f32p, _f32p, _sz, _f32p]
    l.qto_relu2_mul.argtypes = [_f32p, _f32p, _sz, _f32p]
    l.qto_expf_restated.restype = C.c_float
    l.qto_expf_restated.argtypes = [C.c_float]
    l.qto_exp2_table.restype = _u64p
    l.qto_attend_head.argtypes = [_f32p, _u16p, _u16p, _sz, _sz, _sz, _sz, C.c_float, C.c_int, _f32p]
    l.qto_argmax.restype = C.c_uint32
    l.qto_argmax.argtypes = [_f32p, _sz]
    l.qto_model_create.restype = C.c_void_p
    l.qto_model_create.argtypes = [C.c_int] * 11 + [C.c_float, C.c_float, _u16p, _u16p, _f32p, C.POINTER(_u8p), _f32p, C.POINTER(_f32p)]
    l.qto_model_free.argtypes = [C.c_void_p]
    l.qto_model_forward.argtypes = [C.c_void_p, C.c_uint32, _sz, _f32p]
    l.qto_model_set_bf16_tables.argtypes = [C.c_void_p, C.c_int]
    l.qto_model_set_block_scales.argtypes = [C.c_void_p, C.POINTER(_f32p)]
    l.qto_model_set_qk_norms.argtypes = [C.c_void_p, C.POINTER(_f32p)]
    l.qto_vec_dot_bf16.restype = C.c_float
    l.qto_vec_dot_bf16.argtypes = [_u16p, _u16p, _sz]
    l.qto_f32_to_bf16.restype = C.c_uint16
    l.qto_f32_to_bf16.argtypes = [C.c_float]
    l.qto_quantize_q8_0.argtypes = [_f32p, _sz, _i8p, _f32p]
    l.qto_block_scaled_dot_row.restype = C.c_float
    l.qto_block_scaled_dot_row.argtypes = [_u8p, _f32p, _i8p, _f32p, _sz]
    l.qto_block_scaled_dot_trits.restype = C.c_float
    l.qto_block_scaled_dot_trits.argtypes = [_i8p, _f32p, _i8p, _f32p, _sz]
    l.qto_gemv_block_scaled.argtypes = [_u8p, _f32p, _i8p, _f32p, _sz, _sz, _f32p]
    l.qto_fast_enable.argtypes = [C.c_int]
    l.qto_fast_available.restype = C.c_int


_model_declared = False


def mlib() -> C.CDLL:
    global _model_declared
    l = lib()
    if not _model_declared:
        _declare_model(l)
        _model_declared = True
    return l


def f32_to_f16_bits(x) -> np.ndarray:
    xx = _c(x, np.float32).reshape(-1)
    l = mlib()
    return np.array([l.qto_f32_to_f16(float(v)) for v in xx], np.uint16)


def rms_norm(x, w, eps: float) -> np.ndarray:
    xx, ww = _c(x, np.float32), _c(w, np.float32)
    out = np.zeros(xx.size, np.float32)
    mlib().qto_rms_norm(_p(xx, _f32p), _p(ww, _f32p), xx.size, eps, _p(out, _f32p))
    return out


def rope_cache(pos: int, n_dims: int, freq_base: float) -> np.ndarray:
    out = np.zeros(n_dims, np.float32)
    mlib().qto_rope_cache(pos, n_dims, freq_base, _p(out, _f32p))
    return out


def rope_apply(x, heads: int, head_dim: int, mode: int, cache) -> np.ndarray:
    xx = _c(x, np.float32).copy()
    cc = _c(cache, np.float32)
    mlib().qto_rope_apply(_p(xx, _f32p), heads, head_dim, mode, _p(cc, _f32p), cc.size)
    return xx


def vec_dot_f16(x, y) -> np.float32:
    a, b = _c(x, np.uint16), _c(y, np.uint16)
    return np.float32(mlib().qto_vec_dot_f16(_p(a, _u16p), _p(b, _u16p), a.size))


def vec_dot_f16_f32(x, y) -> np.float32:
    a, b = _c(x, np.uint16), _c(y, np.float32)
    return np.float32(mlib().qto_vec_dot_f16_f32(_p(a, _u16p), _p(b, _f32p), a.size))


def swiglu(gate, up) -> np.ndarray:
    g, u = _c(gate, np.float32), _c(up, np.float32)
    out = np.zeros(g.size, np.float32)
    mlib().qto_swiglu(_p(g, _f32p), _p(u, _f32p), g.size, _p(out, _f32p))
    return out


def relu2_mul(gate, up) -> np.ndarray:
    g, u = _c(gate, np.float32), _c(up, np.float32)
    out = np.zeros(g.size, np.float32)
    mlib().qto_relu2_mul(_p(g, _f32p), _p(u, _f32p), g.size, _p(out, _f32p))
    return out


def expf_restated(x) -> np.ndarray:
    xx = _c(x, np.float32).reshape(-1)
    l = mlib()
    return np.array([l.qto_expf_restated(float(v)) for v in xx], np.float32)


def exp2_table() -> np.ndarray:
    return np.ctypeslib.as_array(mlib().qto_exp2_table(), shape=(32,)).copy()


def attend_head(q, k, v, stride: int, seq_len: int, max_seq_len: int, head_dim: int, scale: float, f32_values: bool) -> np.ndarray:
    qq, kk, vv = _c(q, np.float32), _c(k, np.uint16).reshape(-1), _c(v, np.uint16).reshape(-1)
    out = np.zeros(head_dim, np.float32)
    mlib().qto_attend_head(_p(qq, _f32p), _p(kk, _u16p), _p(vv, _u16p), stride, seq_len, max_seq_len, head_dim, scale, int(f32_values), _p(out, _f32p))
    return out


def argmax(logits) -> int:
    x = _c(logits, np.float32)
    return int(mlib().qto_argmax(_p(x, _f32p), x.size))


class Model:
    """Whole-token CPU forward over a model given as numpy arrays (see quintrit_b200.synth.make_model)."""

    def __init__(self, spec: dict):
        l = mlib()
        self.spec = spec
        L = spec["layers"]
        self._keep = []
        w = (_u8p * (L * 7))()
        for i, a in enumerate(spec["weights"]):
            a = _c(a, np.uint8)
            self._keep.append(a)
            w[i] = _p(a, _u8p)
        norms = (_f32p * (L * 4))()
        for i, a in enumerate(spec["norms"]):
            if a is None:
                norms[i] = None
            else:
                a = _c(a, np.float32)
                self._keep.append(a)
                norms[i] = _p(a, _f32p)
        scales = _c(spec["scales"], np.float32)
        embed = _c(spec["embed"], np.uint16)
        head = None if spec.get("lm_head") is None else _c(spec["lm_head"], np.uint16)
        out_norm = _c(spec["out_norm"], np.float32)
        self._keep += [scales, embed, head, out_norm, w, norms]
        self._h = l.qto_model_create(spec["arch"], int(spec["f32_values"]), spec["hidden"], spec["inter"], L, spec["q_heads"], spec["kv_heads"],
                                     spec["head_dim"], spec["vocab"], spec["ctx"], spec["rope_dims"], spec["eps"], spec["rope_theta"],
                                     _p(embed, _u16p), None if head is None else _p(head, _u16p), _p(out_norm, _f32p), w, _p(scales, _f32p), norms)
        if spec.get("bf16_tables"):
            l.qto_model_set_bf16_tables(self._h, 1)
        if spec.get("block_scales") is not None:  # Q2_0 model: layers * 7 arrays of per-64-weight scales
            bsc = (_f32p * (L * 7))()
            for i, a in enumerate(spec["block_scales"]):
                a = _c(a, np.float32)
                self._keep.append(a)
                bsc[i] = _p(a, _f32p)
            self._keep.append(bsc)
            l.qto_model_set_block_scales(self._h, bsc)

        if spec.get("qk_norms") is not None:  # layers * 2 arrays of head_dim weights (query norm, key norm)
            qkn = (_f32p * (L * 2))()
            for i, a in enumerate(spec["qk_norms"]):
                a = _c(a, np.float32)
                self._keep.append(a)
                qkn[i] = _p(a, _f32p)
            self._keep.append(qkn)
            l.qto_model_set_qk_norms(self._h, qkn)

    def forward(self, token: int, pos: int) -> np.ndarray:
        logits = np.zeros(self.spec["vocab"], np.float32)
        mlib().qto_model_forward(self._h, token, pos, _p(logits, _f32p))
        return logits

    def __del__(self):
        try:
            mlib().qto_model_free(self._h)
        except Exception:
            pass


def quantize_q8_0(x):
    """(codes int8[n], block scales f32[n/32]) of ops.rs:898-910; n must be a multiple of 32."""
    xx = _c(x, np.float32).reshape(-1)
    assert xx.size % 32 == 0
    qs, d = np.zeros(xx.size, np.int8), np.zeros(xx.size // 32, np.float32)
    mlib().qto_quantize_q8_0(_p(xx, _f32p), xx.size, _p(qs, _i8p), _p(d, _f32p))
    return qs, d


def block_scaled_dot_row(row, w_scales, acts, a_scales, cols: int) -> np.float32:
    r, ws, a, sc = _c(row, np.uint8), _c(w_scales, np.float32), _c(acts, np.int8), _c(a_scales, np.float32)
    return np.float32(mlib().qto_block_scaled_dot_row(_p(r, _u8p), _p(ws, _f32p), _p(a, _i8p), _p(sc, _f32p), cols))


def block_scaled_dot_trits(trits, w_scales, acts, a_scales, cols: int) -> np.float32:
    t, ws, a, sc = _c(trits, np.int8), _c(w_scales, np.float32), _c(acts, np.int8), _c(a_scales, np.float32)
    return np.float32(mlib().qto_block_scaled_dot_trits(_p(t, _i8p), _p(ws, _f32p), _p(a, _i8p), _p(sc, _f32p), cols))


def gemv_block_scaled(planar, w_scales, acts, a_scales, rows: int, cols: int) -> np.ndarray:
    pl, ws, a, sc = _c(planar, np.uint8), _c(w_scales, np.float32), _c(acts, np.int8), _c(a_scales, np.float32)
    out = np.zeros(rows, np.float32)
    mlib().qto_gemv_block_scaled(_p(pl, _u8p), _p(ws, _f32p), _p(a, _i8p), _p(sc, _f32p), rows, cols, _p(out, _f32p))
    return out


def vec_dot_bf16(x, y) -> np.float32:
    """ggml_vec_dot_bf16 (ops.rs:688-712) of two vectors given as BF16 bit patterns."""
    xx, yy = _c(x, np.uint16), _c(y, np.uint16)
    return np.float32(mlib().qto_vec_dot_bf16(_p(xx, _u16p), _p(yy, _u16p), xx.size))


def f32_to_bf16_bits(x) -> np.ndarray:
    xx = _c(x, np.float32).reshape(-1)
    l = mlib()
    return np.array([l.qto_f32_to_bf16(float(v)) for v in xx], np.uint16)
