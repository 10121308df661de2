"""Test infrastructure: the reference's own CUDA kernels (rust/crates/quintrit-cuda/kernels/gemv.cu, layer.cu) behind the host
launchers of oracle/ref_cuda/ref_launcher.cu, built into oracle/_ref/libqtref_cuda.so by oracle/ref_cuda/Makefile where the
reference tree is available. The built library travels to the GPU machine; the sources stay in the reference tree. Used by the
GPU tests (the oracle and the library against the code they restate and replace) and by the benchmark's reference-cuda arm.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "libqtref_cuda.so")
_lib = None


def build(reference: str) -> str:
    """Compiles the reference's kernels from `reference` (the root of the reference tree); raises if nvcc fails."""
    r = subprocess.run(["make", "-C", os.path.join(HERE, "ref_cuda"), f"REF={os.path.abspath(reference)}"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the reference's CUDA kernels failed:\n" + r.stdout + r.stderr)
    return LIB


def available() -> bool:
    return os.path.exists(LIB)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        l = C.CDLL(LIB)
        l.qtref_config_tag.restype = C.c_char_p
        l.qtref_act_perm_bytes.restype = C.c_size_t
        vp, i = C.c_void_p, C.c_int
        l.qtref_gemv_plain.argtypes = [i, vp, i, i, vp, vp]
        l.qtref_gemv_plain_device.argtypes = [i, vp, i, i, vp, vp, vp, vp]
        l.qtref_permute_activations.argtypes = [vp, i, vp, C.c_size_t, C.POINTER(C.c_int)]
        l.qtref_gemv_gated.argtypes = [i, vp, i, i, vp, C.c_float, C.c_float, C.c_float, i, vp, C.POINTER(C.c_float)]
        l.qtref_rms_quant.argtypes = [vp, vp, i, C.c_float, i, vp, C.POINTER(C.c_float), C.POINTER(C.c_int)]
        l.qtref_head.argtypes = [vp, vp, vp, i, i, C.c_float, vp, vp]
        l.qtref_rope_kv.argtypes = [vp, C.c_float, C.c_float, C.c_float, C.c_float, vp, i, i, i, i, i, i, vp, vp, vp]
        l.qtref_attention.argtypes = [vp, vp, vp, i, i, i, i, i, C.c_float, vp]
        _lib = l
    return _lib


def _ok(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: CUDA error {rc}")


def _a(x, dtype) -> np.ndarray:
    return np.ascontiguousarray(x, dtype)


def configs() -> list[tuple[int, str, int]]:
    l = lib()
    return [(k, l.qtref_config_tag(k).decode(), l.qtref_config_rows_per_block(k)) for k in range(l.qtref_config_count())]


def profile_config(role: int) -> int:
    return lib().qtref_profile_config(role)


def gemv_plain(cfg: int, planar, rows: int, cols: int, act) -> np.ndarray:
    w, a, out = _a(planar, np.uint8), _a(act, np.int8), np.zeros(rows, np.int32)
    _ok(lib().qtref_gemv_plain(cfg, w.ctypes.data, rows, cols, a.ctypes.data, out.ctypes.data), "gemv_plain")
    return out


def permute_activations(act) -> tuple[np.ndarray, int]:
    a = _a(act, np.int8)
    out, s = np.zeros(lib().qtref_act_perm_bytes(a.size), np.int8), C.c_int(0)
    _ok(lib().qtref_permute_activations(a.ctypes.data, a.size, out.ctypes.data, out.size, C.byref(s)), "permute")
    return out, s.value


def gemv_gated(cfg: int, interleaved, rows: int, cols: int, act, act_scale: float, ws_gate: float, ws_up: float, activation: int):
    w, a, v, amax = _a(interleaved, np.uint8), _a(act, np.int8), np.zeros(rows // 2, np.float32), C.c_float(0)
    _ok(lib().qtref_gemv_gated(cfg, w.ctypes.data, rows, cols, a.ctypes.data, act_scale, ws_gate, ws_up, activation, v.ctypes.data, C.byref(amax)), "gemv_gated")
    return v, np.float32(amax.value)


def rms_quant(x, gamma, eps: float, norm: bool = True):
    xx, g = _a(x, np.float32), _a(gamma, np.float32)
    q, s, total = np.zeros(xx.size, np.int8), C.c_float(0), C.c_int(0)
    _ok(lib().qtref_rms_quant(xx.ctypes.data, g.ctypes.data, xx.size, eps, int(norm), q.ctypes.data, C.byref(s), C.byref(total)), "rms_quant")
    return q, np.float32(s.value), total.value


def head(h, norm_w, head_f16, vocab: int, eps: float):
    hh, w, W = _a(h, np.float32), _a(norm_w, np.float32), _a(head_f16, np.uint16)
    normed, logits = np.zeros(hh.size, np.float32), np.zeros(vocab, np.float32)
    _ok(lib().qtref_head(hh.ctypes.data, w.ctypes.data, W.ctypes.data, vocab, hh.size, eps, normed.ctypes.data, logits.ctypes.data), "head")
    return normed, logits


def rope_kv(qkv, act_scale, ws_q, ws_k, ws_v, cos_sin, pos, q_heads, kv_heads, head_dim, rope_dims, neox):
    x, cs = _a(qkv, np.int32), _a(cos_sin, np.float32)
    q, k, v = np.zeros(q_heads * head_dim, np.float32), np.zeros(kv_heads * head_dim, np.uint16), np.zeros(kv_heads * head_dim, np.uint16)
    _ok(lib().qtref_rope_kv(x.ctypes.data, act_scale, ws_q, ws_k, ws_v, cs.ctypes.data, pos, q_heads, kv_heads, head_dim, rope_dims, int(neox), q.ctypes.data, k.ctypes.data,
                            v.ctypes.data), "rope_kv")
    return q, k, v


def attention(K, V, q, q_heads: int, kv_heads: int, head_dim: int, cache_len: int, pos: int, scale: float) -> np.ndarray:
    """K, V: [kv_heads][cache_len][head_dim] F16 bit patterns; q: [q_heads][head_dim]."""
    kk, vv, qq, out = _a(K, np.uint16), _a(V, np.uint16), _a(q, np.float32), np.zeros(q_heads * head_dim, np.float32)
    _ok(lib().qtref_attention(kk.ctypes.data, vv.ctypes.data, qq.ctypes.data, q_heads, kv_heads, head_dim, cache_len, pos, scale, out.ctypes.data), "attention")
    return out
