"""ctypes host side of ``libquintrit_b200.so``.

Names follow the reference's GPU crate: ``pack_planar`` / ``row_bytes`` (``rust/crates/quintrit-cuda/src/pack.rs:24-48``),
``Matrix`` = an uploaded ``DeviceBuffer<u8>`` of planar weights plus its shape, ``Matrix.gemv_i32`` = ``Gemv::plain``
(``rust/crates/quintrit-cuda/src/gemv.rs:191-226``) with upload and download, ``Matrix.forward`` =
``TernaryGemvLayer::forward`` (``rust/crates/quintrit-runtime/src/layer.rs:123-177``).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from . import build as _build

SRC_PLANAR, SRC_TQ1_0, SRC_TQ2_0, SRC_I2_S, SRC_Q2_0 = 0, 34, 35, 36, 42

_u8p, _i8p, _i32p, _f32p = (C.POINTER(t) for t in (C.c_uint8, C.c_int8, C.c_int32, C.c_float))
_sz = C.c_size_t
_lib = None


class QuintritError(RuntimeError):
    """A call into the C ABI returned a status other than QUINTRIT_OK."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


class _DeviceInfoC(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("index", C.c_uint32), ("compute_major", C.c_int32), ("compute_minor", C.c_int32),
                ("sm_count", C.c_uint32), ("supported", C.c_uint32), ("total_memory", C.c_uint64), ("l2_cache_bytes", C.c_uint64),
                ("name", C.c_char * 64)]


class _GpuOptionsC(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("device_index", C.c_uint32), ("context_length", C.c_uint32), ("flags", C.c_uint32)]


class _DecoderInfoC(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("arch", C.c_int32), ("f32_values", C.c_int32)] + [
        (n, C.c_uint32) for n in ("hidden_size", "intermediate_size", "num_layers", "num_heads", "num_kv_heads", "head_dim", "vocab_size",
                                  "context_length", "rope_dims", "device_index", "single_kernel", "table_dtype")]


class _DecoderDescC(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("device_index", C.c_uint32), ("arch", C.c_int32), ("f32_values", C.c_int32),
                ("hidden_size", C.c_uint32), ("intermediate_size", C.c_uint32), ("num_layers", C.c_uint32), ("num_heads", C.c_uint32),
                ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("vocab_size", C.c_uint32), ("context_length", C.c_uint32),
                ("rope_dims", C.c_uint32), ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float), ("embed", C.POINTER(C.c_uint16)),
                ("lm_head", C.POINTER(C.c_uint16)), ("output_norm", _f32p), ("matrices", C.POINTER(C.c_void_p)), ("scales", _f32p),
                ("norms", C.POINTER(_f32p)), ("tp_rank", C.c_uint32), ("tp_world", C.c_uint32), ("table_dtype", C.c_uint32),
                ("qk_norms", C.POINTER(_f32p))]


@dataclass
class DeviceInfo:
    index: int
    compute_major: int
    compute_minor: int
    sm_count: int
    supported: bool
    total_memory: int
    l2_cache_bytes: int
    name: str


def library_path() -> str:
    return _build.LIB


def load_library(build_if_missing: bool = True) -> C.CDLL:
    """Loads the CUDA library; raises if it is absent and cannot be built (there is no fallback path)."""
    global _lib
    if _lib is not None:
        return _lib
    if build_if_missing and _build.needs_build():
        _build.build()
    if not os.path.exists(_build.LIB):
        raise QuintritError(6, f"{_build.LIB} is missing: build it with `python -m quintrit_b200.build`")
    l = C.CDLL(_build.LIB)
    l.quintrit_status_string.restype = C.c_char_p
    l.quintrit_last_error_message.restype = C.c_char_p
    l.quintrit_b200_version.restype = C.c_char_p
    l.quintrit_b200_abi_version.restype = C.c_uint32
    l.quintrit_cuda_device_count.argtypes = [C.POINTER(C.c_uint32)]
    l.quintrit_cuda_device_info.argtypes = [C.c_uint32, C.POINTER(_DeviceInfoC)]
    l.quintrit_b200_planar_row_bytes.restype = _sz
    l.quintrit_b200_planar_row_bytes.argtypes = [_sz]
    l.quintrit_b200_pack_planar.argtypes = [_i8p, _sz, _sz, _sz, _u8p, _sz]
    l.quintrit_b200_matrix_upload.argtypes = [C.c_uint32, C.c_int32, _u8p, _sz, _sz, _sz, C.POINTER(C.c_void_p)]
    l.quintrit_b200_matrix_free.argtypes = [C.c_void_p]
    l.quintrit_b200_matrix_info.argtypes = [C.c_void_p, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz)]
    l.quintrit_b200_matrix_download_planar.argtypes = [C.c_void_p, _u8p, _sz]
    l.quintrit_b200_matrix_scales.argtypes = [C.c_void_p, _f32p, _sz]
    l.quintrit_b200_quantize_q8_0.argtypes = [C.c_uint32, _f32p, _sz, _i8p, _f32p]
    l.quintrit_b200_gemv_block_scaled.argtypes = [C.c_void_p, _f32p, _sz, _f32p, _sz]
    l.quintrit_b200_gemv_block_scaled_q8.argtypes = [C.c_void_p, _i8p, _sz, _f32p, _sz, _f32p, _sz]
    l.quintrit_b200_gemv_i32.argtypes = [C.c_void_p, _i8p, _sz, _i32p, _sz]
    l.quintrit_b200_gemv_f32.argtypes = [C.c_void_p, _i8p, _sz, C.c_float, _f32p, _sz]
    l.quintrit_b200_gemm_i32.argtypes = [C.c_void_p, _i8p, _sz, _sz, _i32p, _sz]
    l.quintrit_b200_gemm_i32_device.argtypes = [C.c_void_p, C.c_void_p, _sz, C.c_void_p, C.c_void_p]
    l.quintrit_b200_gemv_i32_device.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    l.quintrit_b200_gemv_i32_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    l.quintrit_b200_plan_create.argtypes = [C.POINTER(C.c_void_p), _sz, C.POINTER(C.c_void_p)]
    l.quintrit_b200_plan_free.argtypes = [C.c_void_p]
    l.quintrit_b200_plan_layout.argtypes = [C.c_void_p, _sz, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz)]
    l.quintrit_b200_plan_buffers.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]
    l.quintrit_b200_plan_launch.argtypes = [C.c_void_p, C.c_void_p]
    l.quintrit_b200_plan_run.argtypes = [C.c_void_p, _i8p, _sz, _i32p, _sz]
    l.quintrit_b200_decoder_create.argtypes = [C.POINTER(_DecoderDescC), C.POINTER(C.c_void_p)]
    l.quintrit_b200_decoder_free.argtypes = [C.c_void_p]
    l.quintrit_b200_decoder_tp_handle.argtypes = [C.c_void_p, _u8p, _sz]
    l.quintrit_b200_decoder_tp_attach.argtypes = [C.c_void_p, _u8p, _sz]
    l.quintrit_b200_decoder_tp_attach_local.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), _sz]
    l.quintrit_b200_decoder_open_gguf.argtypes = [C.c_char_p, C.POINTER(_GpuOptionsC), C.POINTER(C.c_void_p)]
    l.quintrit_b200_decoder_info.argtypes = [C.c_void_p, C.POINTER(_DecoderInfoC)]
    l.quintrit_b200_gguf_describe.argtypes = [C.c_char_p, C.c_char_p, _sz, C.POINTER(_sz)]
    l.quintrit_b200_decoder_forward.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, _f32p, _sz, C.POINTER(C.c_uint32)]
    l.quintrit_b200_decoder_prefill.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), _sz, C.c_uint32, _f32p, _sz, C.POINTER(C.c_uint32)]
    _u32p = C.POINTER(C.c_uint32)
    l.quintrit_b200_batch_create.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(C.c_void_p)]
    l.quintrit_b200_batch_free.argtypes = [C.c_void_p]
    l.quintrit_b200_batch_free.restype = None
    l.quintrit_b200_batch_info.argtypes = [C.c_void_p, _u32p, _u32p, _u32p, _sz]
    l.quintrit_b200_batch_rewind.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32]
    l.quintrit_b200_batch_prefill.argtypes = [C.c_void_p, C.c_uint32, _u32p, _sz, _f32p, _sz, _u32p]
    l.quintrit_b200_batch_step.argtypes = [C.c_void_p, _u32p, _sz, _u32p, _u32p, _f32p, _sz]
    l.quintrit_b200_decoder_generate.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), _sz, _sz, C.POINTER(C.c_uint32), _sz]
    l.quintrit_b200_decoder_time_token.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(C.c_float)]
    l.quintrit_b200_decoder_trace_step.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), _sz, C.POINTER(_sz)]
    l.quintrit_b200_selftest_barrier.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32)]
    l.quintrit_b200_launch_count.restype = C.c_uint64
    l.quintrit_b200_launch_count.argtypes = [C.c_int]
    _lib = l
    return l


def _check(rc: int) -> None:
    if rc != 0:
        raise QuintritError(rc, load_library().quintrit_last_error_message().decode("utf-8", "replace"))


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def version() -> str:
    return load_library().quintrit_b200_version().decode()


def device_count() -> int:
    n = C.c_uint32(0)
    _check(load_library().quintrit_cuda_device_count(C.byref(n)))
    return n.value


def device_info(index: int = 0) -> DeviceInfo:
    info = _DeviceInfoC()
    info.struct_size = C.sizeof(_DeviceInfoC)
    _check(load_library().quintrit_cuda_device_info(index, C.byref(info)))
    return DeviceInfo(info.index, info.compute_major, info.compute_minor, info.sm_count, bool(info.supported), info.total_memory,
                      info.l2_cache_bytes, info.name.decode("utf-8", "replace"))


def launch_count(reset: bool = False) -> int:
    return int(load_library().quintrit_b200_launch_count(1 if reset else 0))


_selftest_released = 0


def selftest_barrier(device: int = 0, ctas: int = 4, spin_limit: int = 5000) -> int:
    """Runs the barrier's give-up self-test (quintrit_b200_selftest_barrier). The expected outcome is a QuintritError with
    code 15; the number of CTAs the failure released is kept for last_selftest_released()."""
    global _selftest_released
    n = C.c_uint32(0)
    rc = load_library().quintrit_b200_selftest_barrier(device, ctas, spin_limit, C.byref(n))
    _selftest_released = n.value
    _check(rc)
    return n.value


def last_selftest_released() -> int:
    return _selftest_released


def row_bytes(cols: int) -> int:
    """Bytes of one planar row (quintrit-cuda/src/pack.rs:29-32)."""
    return int(load_library().quintrit_b200_planar_row_bytes(cols))


def pack_planar(trits, rows: int, cols: int) -> np.ndarray:
    """rows x cols trits -> planar velurex bytes (quintrit-cuda/src/pack.rs:42-48)."""
    t = np.ascontiguousarray(trits, dtype=np.int8).reshape(-1)
    out = np.zeros(rows * row_bytes(cols), np.uint8)
    _check(load_library().quintrit_b200_pack_planar(_p(t, _i8p), t.size, rows, cols, _p(out, _u8p), out.size))
    return out


class Matrix:
    """A ternary matrix resident in HBM in the stream layout."""

    def __init__(self, data, rows: int, cols: int, source: int = SRC_PLANAR, device: int = 0):
        d = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
        h = C.c_void_p()
        _check(load_library().quintrit_b200_matrix_upload(device, source, _p(d, _u8p), d.size, rows, cols, C.byref(h)))
        self._h, self.rows, self.cols, self.device = h, rows, cols, device

    @classmethod
    def from_trits(cls, trits, rows: int, cols: int, device: int = 0) -> "Matrix":
        return cls(pack_planar(trits, rows, cols), rows, cols, SRC_PLANAR, device)

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    @property
    def device_bytes(self) -> int:
        n = _sz(0)
        _check(load_library().quintrit_b200_matrix_info(self._h, None, None, C.byref(n)))
        return n.value

    def download_planar(self) -> np.ndarray:
        out = np.zeros(self.rows * row_bytes(self.cols), np.uint8)
        _check(load_library().quintrit_b200_matrix_download_planar(self._h, _p(out, _u8p), out.size))
        return out

    def scales(self) -> np.ndarray:
        """The per-64-weight scales of a block-scaled (Q2_0) matrix, row-major."""
        out = np.zeros(self.rows * (self.cols // 64), np.float32)
        _check(load_library().quintrit_b200_matrix_scales(self._h, _p(out, _f32p), out.size))
        return out

    def gemv_block_scaled(self, x) -> np.ndarray:
        """``quantize_q8_0`` + ``BlockScaledLayer::forward_q8`` for f32 activations (Q2_0 matrices)."""
        xx = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros(self.rows, np.float32)
        _check(load_library().quintrit_b200_gemv_block_scaled(self._h, _p(xx, _f32p), xx.size, _p(out, _f32p), out.size))
        return out

    def gemv_block_scaled_q8(self, codes, scales) -> np.ndarray:
        """``BlockScaledLayer::forward_q8`` for activations that are Q8_0 blocks already."""
        q, d = np.ascontiguousarray(codes, dtype=np.int8), np.ascontiguousarray(scales, dtype=np.float32)
        out = np.zeros(self.rows, np.float32)
        _check(load_library().quintrit_b200_gemv_block_scaled_q8(self._h, _p(q, _i8p), q.size, _p(d, _f32p), d.size, _p(out, _f32p), out.size))
        return out

    def gemm_i32(self, activations) -> np.ndarray:
        """Batched projection on the tensor cores: activations [batch, cols] int8 -> [batch, rows] int32, every row the integers of gemv_i32."""
        a = np.ascontiguousarray(activations, dtype=np.int8).reshape(-1, self.cols)
        out = np.zeros((a.shape[0], self.rows), np.int32)
        _check(load_library().quintrit_b200_gemm_i32(self._h, _p(a, _i8p), a.size, a.shape[0], _p(out, _i32p), out.size))
        return out

    def gemm_i32_device(self, d_activations: int, batch: int, d_out: int, stream: int = 0) -> None:
        _check(load_library().quintrit_b200_gemm_i32_device(self._h, d_activations, batch, d_out, stream))

    def gemv_i32(self, activations) -> np.ndarray:
        a = np.ascontiguousarray(activations, dtype=np.int8)
        out = np.zeros(self.rows, np.int32)
        _check(load_library().quintrit_b200_gemv_i32(self._h, _p(a, _i8p), a.size, _p(out, _i32p), out.size))
        return out

    def gemv_f32(self, activations, scale: float) -> np.ndarray:
        a = np.ascontiguousarray(activations, dtype=np.int8)
        out = np.zeros(self.rows, np.float32)
        _check(load_library().quintrit_b200_gemv_f32(self._h, _p(a, _i8p), a.size, scale, _p(out, _f32p), out.size))
        return out

    def forward(self, activations, act_scale: float, weight_scale: float) -> np.ndarray:
        """``TernaryGemvLayer::forward``: acc * (weight_scale / act_scale), zeros when act_scale <= 0."""
        if not act_scale > 0:
            return np.zeros(self.rows, np.float32)
        return self.gemv_f32(activations, float(np.float32(weight_scale) / np.float32(act_scale)))

    def gemv_i32_device(self, d_activations: int, d_out: int, stream: int = 0) -> None:
        _check(load_library().quintrit_b200_gemv_i32_device(self._h, C.c_void_p(d_activations), C.c_void_p(d_out), C.c_void_p(stream)))

    def gemv_i32_noalloc(self, d_activations: int, d_out: int, stream: int = 0) -> None:
        """The same GEMV on device pointers through the entry point that allocates nothing (its scratch is a static
        device array shared by all calls on the GPU: do not overlap two of these calls)."""
        _check(load_library().quintrit_b200_gemv_i32_noalloc(self._h, C.c_void_p(d_activations), C.c_void_p(d_out), C.c_void_p(stream)))

    def free(self) -> None:
        if self._h:
            load_library().quintrit_b200_matrix_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Plan:
    """Several GEMVs run as one persistent launch (one decode step's projections)."""

    def __init__(self, matrices):
        self.matrices = list(matrices)
        arr = (C.c_void_p * len(self.matrices))(*[m.handle for m in self.matrices])
        h = C.c_void_p()
        _check(load_library().quintrit_b200_plan_create(arr, len(self.matrices), C.byref(h)))
        self._h = h
        ao, oo, at, ot = _sz(), _sz(), _sz(), _sz()
        self.act_offsets, self.out_offsets = [], []
        for i in range(len(self.matrices)):
            _check(load_library().quintrit_b200_plan_layout(h, i, C.byref(ao), C.byref(oo), C.byref(at), C.byref(ot)))
            self.act_offsets.append(ao.value)
            self.out_offsets.append(oo.value)
        self.act_total, self.out_total = at.value, ot.value

    def pack_activations(self, acts) -> np.ndarray:
        buf = np.zeros(self.act_total, np.int8)
        for off, m, a in zip(self.act_offsets, self.matrices, acts):
            buf[off:off + m.cols] = a
        return buf

    def split_results(self, out: np.ndarray):
        return [out[off:off + m.rows] for off, m in zip(self.out_offsets, self.matrices)]

    def buffers(self):
        a, o = C.c_void_p(), C.c_void_p()
        _check(load_library().quintrit_b200_plan_buffers(self._h, C.byref(a), C.byref(o)))
        return a.value, o.value

    def launch(self, stream: int = 0) -> None:
        _check(load_library().quintrit_b200_plan_launch(self._h, C.c_void_p(stream)))

    def run(self, activations: np.ndarray, out: np.ndarray | None = None) -> np.ndarray:
        a = np.ascontiguousarray(activations, dtype=np.int8)
        if out is None:
            out = np.zeros(self.out_total, np.int32)
        _check(load_library().quintrit_b200_plan_run(self._h, _p(a, _i8p), a.size, _p(out, _i32p), out.size))
        return out

    def free(self) -> None:
        if self._h:
            load_library().quintrit_b200_plan_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


ARCH_LLAMA, ARCH_BITNET, ARCH_QWEN = 0, 1, 2


class Decoder:
    """Whole-token decoder on the device: ``GpuModel`` + ``GpuSession`` of ``rust/crates/quintrit-runtime/src/gpu.rs``.

    ``spec`` is a dict as made by ``quintrit_b200.synth.make_model``: dimensions, ``weights`` (layers * 7 planar byte
    arrays in the order q, k, v, o, gate, up, down, or ``(source, payload)`` pairs for GGUF encodings), ``scales``,
    ``norms`` (layers * 4, None where absent), ``embed`` / ``lm_head`` as F16 bit patterns, ``out_norm``.
    """

    def __init__(self, spec: dict, device: int = 0):
        self.spec = spec
        L, H, I, hd = spec["layers"], spec["hidden"], spec["inter"], spec["head_dim"]
        qd, kvd = spec["q_heads"] * hd, spec["kv_heads"] * hd
        self.tp_rank, self.tp_world = spec.get("tp_rank", 0), spec.get("tp_world", 1)
        w = self.tp_world  # a rank of a tensor-parallel group holds its rows of every projection (synth.shard_spec)
        hw = w if spec["kv_heads"] % w == 0 else 1  # ranks that do not divide the KV heads hold q, k and v whole (attention is replicated)
        shapes = [(qd // hw, H), (kvd // hw, H), (kvd // hw, H), (H // w, qd), (I // w, H), (I // w, H), (H // w, I)]
        self.matrices = []
        for i, w in enumerate(spec["weights"]):
            rows, cols = shapes[i % 7]
            if isinstance(w, tuple):
                self.matrices.append(Matrix(w[1], rows, cols, source=w[0], device=device))
            else:
                self.matrices.append(Matrix(w, rows, cols, device=device))
        keep = []
        mats = (C.c_void_p * (L * 7))(*[m.handle for m in self.matrices])
        norms = (_f32p * (L * 4))()
        for i, a in enumerate(spec["norms"]):
            if a is not None:
                a = np.ascontiguousarray(a, np.float32)
                keep.append(a)
                norms[i] = _p(a, _f32p)
        scales = np.ascontiguousarray(spec["scales"], np.float32)
        embed = np.ascontiguousarray(spec["embed"], np.uint16)
        head = None if spec.get("lm_head") is None else np.ascontiguousarray(spec["lm_head"], np.uint16)
        out_norm = np.ascontiguousarray(spec["out_norm"], np.float32)
        d = _DecoderDescC()
        d.struct_size = C.sizeof(_DecoderDescC)
        d.device_index, d.arch, d.f32_values = device, spec["arch"], int(spec["f32_values"])
        d.hidden_size, d.intermediate_size, d.num_layers = H, I, L
        d.num_heads, d.num_kv_heads, d.head_dim = spec["q_heads"], spec["kv_heads"], hd
        d.vocab_size, d.context_length, d.rope_dims = spec["vocab"], spec["ctx"], spec["rope_dims"]
        d.rms_norm_eps, d.rope_theta = spec["eps"], spec["rope_theta"]
        d.embed = _p(embed, C.POINTER(C.c_uint16))
        d.lm_head = None if head is None else _p(head, C.POINTER(C.c_uint16))
        d.output_norm = _p(out_norm, _f32p)
        d.matrices, d.scales, d.norms = mats, _p(scales, _f32p), norms
        d.tp_rank, d.tp_world = self.tp_rank, self.tp_world
        d.table_dtype = 1 if spec.get("bf16_tables") else 0
        if spec.get("qk_norms") is not None:  # layers * 2 arrays of head_dim weights (query norm, key norm)
            qkn = (_f32p * (L * 2))()
            for i, a in enumerate(spec["qk_norms"]):
                a = np.ascontiguousarray(a, dtype=np.float32)
                keep.append(a)
                qkn[i] = _p(a, _f32p)
            keep.append(qkn)
            d.qk_norms = qkn
        h = C.c_void_p()
        _check(load_library().quintrit_b200_decoder_create(C.byref(d), C.byref(h)))
        self._h = h
        self.vocab = spec["vocab"] // self.tp_world  # logits returned by forward(): this rank's rows of the vocabulary

    def tp_handle(self) -> bytes:
        """The 64-byte inter-process handle of this rank's exchange box (tensor-parallel decoders)."""
        out = np.zeros(64, np.uint8)
        _check(load_library().quintrit_b200_decoder_tp_handle(self._h, _p(out, _u8p), out.size))
        return out.tobytes()

    def tp_attach_local(self, group) -> None:
        """Maps the boxes of a group of decoders that live in this process (rank order, this decoder among them)."""
        hs = (C.c_void_p * len(group))(*[g._h for g in group])
        _check(load_library().quintrit_b200_decoder_tp_attach_local(self._h, hs, len(group)))

    def tp_attach(self, handles) -> None:
        """Maps the boxes of all ranks; `handles` are the tp_handle() bytes of every rank in rank order."""
        raw = np.frombuffer(b"".join(handles), np.uint8).copy()
        _check(load_library().quintrit_b200_decoder_tp_attach(self._h, _p(raw, _u8p), raw.size))

    @classmethod
    def open(cls, path: str, device: int = 0, context: int = 0, flags: int = 0) -> "Decoder":
        """Loads a GGUF model file onto the GPU (``quintrit_model_open_gpu`` without the tokenizer)."""
        self = cls.__new__(cls)
        self.spec, self.matrices = None, []
        opts = _GpuOptionsC(C.sizeof(_GpuOptionsC), device, context, flags)
        h = C.c_void_p()
        _check(load_library().quintrit_b200_decoder_open_gguf(str(path).encode(), C.byref(opts), C.byref(h)))
        self._h = h
        self.vocab = self.info()["vocab_size"]
        return self

    def prefill(self, tokens, pos: int = 0):
        """Ingests `tokens` at positions pos .. in chunks on the tensor cores; returns (logits of the last token, its greedy successor)."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits, nxt = np.zeros(self.vocab, np.float32), C.c_uint32(0)
        _check(load_library().quintrit_b200_decoder_prefill(self._h, t.ctypes.data_as(C.POINTER(C.c_uint32)), t.size, pos, _p(logits, _f32p), logits.size, C.byref(nxt)))
        return logits, nxt.value

    def info(self) -> dict:
        i = _DecoderInfoC()
        i.struct_size = C.sizeof(_DecoderInfoC)
        _check(load_library().quintrit_b200_decoder_info(self._h, C.byref(i)))
        return {n: getattr(i, n) for n, _ in _DecoderInfoC._fields_ if n != "struct_size"}

    def forward(self, token: int, pos: int, want_logits: bool = True):
        """Returns (logits or None, greedy token)."""
        logits = np.zeros(self.vocab, np.float32) if want_logits else None
        tok = C.c_uint32(0)
        _check(load_library().quintrit_b200_decoder_forward(self._h, token, pos, None if logits is None else _p(logits, _f32p),
                                                            0 if logits is None else logits.size, C.byref(tok)))
        return logits, tok.value

    def generate(self, prompt, max_new: int) -> np.ndarray:
        p = np.ascontiguousarray(prompt, np.uint32)
        out = np.zeros(max_new, np.uint32)
        _check(load_library().quintrit_b200_decoder_generate(self._h, _p(p, C.POINTER(C.c_uint32)), p.size, max_new,
                                                             _p(out, C.POINTER(C.c_uint32)), out.size))
        return out

    def trace_step(self) -> np.ndarray:
        """Global-timer stamps (ns) of one decode step at every phase boundary (single-kernel path only)."""
        n = _sz(0)
        load_library().quintrit_b200_decoder_trace_step(self._h, None, 0, C.byref(n))
        out = np.zeros(n.value, np.uint64)
        _check(load_library().quintrit_b200_decoder_trace_step(self._h, _p(out, C.POINTER(C.c_uint64)), out.size, C.byref(n)))
        return out

    def time_token(self, blocks: int = 5, iters: int = 50) -> float:
        ms = C.c_float(0)
        _check(load_library().quintrit_b200_decoder_time_token(self._h, blocks, iters, C.byref(ms)))
        return ms.value

    def free(self) -> None:
        if self._h:
            load_library().quintrit_b200_decoder_free(self._h)
            self._h = C.c_void_p()
        for m in self.matrices:
            m.free()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Batch:
    """Several sequences of one model decoded together (``quintrit_b200_batch_*``): every sequence has its own KV cache and
    position; a step feeds one token per listed sequence through one batched pass over the weights. The decoder must
    outlive the batch and is not used by another thread meanwhile."""

    def __init__(self, decoder: "Decoder", sequences: int):
        self._h = C.c_void_p()
        self.decoder, self.sequences, self.vocab = decoder, sequences, decoder.vocab
        _check(load_library().quintrit_b200_batch_create(decoder._h, sequences, C.byref(self._h)))

    def positions(self) -> np.ndarray:
        out = np.zeros(self.sequences, np.uint32)
        _check(load_library().quintrit_b200_batch_info(self._h, None, None, out.ctypes.data_as(C.POINTER(C.c_uint32)), out.size))
        return out

    def rewind(self, sequence: int, position: int = 0) -> None:
        _check(load_library().quintrit_b200_batch_rewind(self._h, sequence, position))

    def prefill(self, sequence: int, tokens):
        """Appends prompt tokens to one sequence; returns (logits of the last token, its greedy successor)."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits, nxt = np.zeros(self.vocab, np.float32), C.c_uint32(0)
        _check(load_library().quintrit_b200_batch_prefill(self._h, sequence, t.ctypes.data_as(C.POINTER(C.c_uint32)), t.size, _p(logits, _f32p), logits.size,
                                                          C.byref(nxt)))
        return logits, nxt.value

    def step(self, sequences=None, tokens=None, want_logits: bool = False):
        """One token for every listed sequence (all by default), the given tokens or each sequence's last choice; returns
        (greedy tokens, logits [count][vocab] or None)."""
        u32p = C.POINTER(C.c_uint32)
        sq = None if sequences is None else np.ascontiguousarray(sequences, dtype=np.uint32)
        n = self.sequences if sq is None else sq.size
        tk = None if tokens is None else np.ascontiguousarray(tokens, dtype=np.uint32)
        if tk is not None and tk.size != n:
            raise ValueError(f"{tk.size} tokens for {n} sequences")
        out = np.zeros(n, np.uint32)
        logits = np.zeros((n, self.vocab), np.float32) if want_logits else None
        _check(load_library().quintrit_b200_batch_step(self._h, None if sq is None else sq.ctypes.data_as(u32p), n, None if tk is None else tk.ctypes.data_as(u32p),
                                                       out.ctypes.data_as(u32p), None if logits is None else _p(logits, _f32p), 0 if logits is None else logits.size))
        return out, logits

    def free(self) -> None:
        if self._h:
            load_library().quintrit_b200_batch_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Moe:
    """A mixture-of-experts feed-forward block on the GPU (``quintrit_b200_moe_*``): softmax router over BF16 rows, top-k experts, every
    expert a ternary SwiGLU FFN. ``gate_up[e]`` / ``down[e]``: planar velurex rows (gate rows then up rows; down rows), ``scales[e]`` =
    (gate, up, down)."""

    def __init__(self, hidden: int, inter: int, top_k: int, router_bits, gate_up, down, scales, max_batch: int = 16, device: int = 0, n_experts: int | None = None,
                 expert_first: int = 0):
        """With ``n_experts`` larger than ``len(gate_up)`` the block is one GPU's share of an expert-parallel block: it holds the experts
        ``expert_first .. expert_first + len(gate_up) - 1`` (``forward_partial`` / ``pairs_tensor`` / ``finish``)."""
        n = len(gate_up)
        total = n if n_experts is None else n_experts
        self.hidden, self.inter, self.top_k, self.n_experts, self.max_batch = hidden, inter, top_k, total, max_batch
        self._batch = 0
        self.matrices = [Matrix(w, 2 * inter, hidden, device=device) for w in gate_up] + [Matrix(w, hidden, inter, device=device) for w in down]
        gu = (C.c_void_p * n)(*[m.handle for m in self.matrices[:n]])
        dn = (C.c_void_p * n)(*[m.handle for m in self.matrices[n:]])
        rb = np.ascontiguousarray(router_bits, dtype=np.uint16).reshape(-1)
        sc = np.ascontiguousarray(scales, dtype=np.float32).reshape(-1)
        assert rb.size == total * hidden and sc.size == 3 * n
        self._h = C.c_void_p()
        lib = load_library()
        lib.quintrit_b200_moe_create_shard.argtypes = [C.c_uint32] * 6 + [C.POINTER(C.c_uint16), C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _f32p,
                                                       C.POINTER(C.c_void_p)]
        lib.quintrit_b200_moe_forward_partial.argtypes = [C.c_void_p, _f32p, _sz]
        lib.quintrit_b200_moe_pairs.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(_sz)]
        lib.quintrit_b200_moe_finish.argtypes = [C.c_void_p, _sz, _f32p, C.POINTER(C.c_uint32), _f32p]
        lib.quintrit_b200_moe_forward.argtypes = [C.c_void_p, _f32p, _sz, _f32p, C.POINTER(C.c_uint32), _f32p]
        lib.quintrit_b200_moe_time.argtypes = [C.c_void_p, _sz, C.c_uint32, _f32p]
        lib.quintrit_b200_moe_free.argtypes = [C.c_void_p]
        lib.quintrit_b200_moe_free.restype = None
        _check(lib.quintrit_b200_moe_create_shard(device, hidden, inter, total, top_k, max_batch, rb.ctypes.data_as(C.POINTER(C.c_uint16)), expert_first, n, gu, dn, _p(sc, _f32p),
                                                  C.byref(self._h)))

    def forward(self, x):
        """x: [batch][hidden] floats -> (output [batch][hidden], chosen experts [batch][top_k], weights [batch][top_k])."""
        xx = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.hidden)
        b = xx.shape[0]
        out, ids, w = np.zeros((b, self.hidden), np.float32), np.zeros((b, self.top_k), np.uint32), np.zeros((b, self.top_k), np.float32)
        _check(load_library().quintrit_b200_moe_forward(self._h, _p(xx, _f32p), b, _p(out, _f32p), ids.ctypes.data_as(C.POINTER(C.c_uint32)), _p(w, _f32p)))
        return out, ids, w

    def forward_partial(self, x) -> None:
        """Routes the tokens and runs the pairs whose expert this block holds; the pairs' results stay on the device (``pairs_tensor``)."""
        xx = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.hidden)
        self._batch = xx.shape[0]
        _check(load_library().quintrit_b200_moe_forward_partial(self._h, _p(xx, _f32p), self._batch))

    def pairs_tensor(self):
        """The pairs' results of the last partial forward as a torch int32 tensor over the block's device buffer ([batch * top_k * hidden]; the
        bits are floats): the shares of all GPUs are added in place (``torch.distributed.all_reduce``) before ``finish``."""
        import torch

        ptr, n = C.c_void_p(), _sz(0)
        _check(load_library().quintrit_b200_moe_pairs(self._h, C.byref(ptr), C.byref(n)))

        class _View:
            __cuda_array_interface__ = {"shape": (n.value,), "typestr": "<i4", "data": (ptr.value, False), "version": 2}

        return torch.as_tensor(_View(), device="cuda")

    def finish(self):
        b = self._batch
        out, ids, w = np.zeros((b, self.hidden), np.float32), np.zeros((b, self.top_k), np.uint32), np.zeros((b, self.top_k), np.float32)
        _check(load_library().quintrit_b200_moe_finish(self._h, b, _p(out, _f32p), ids.ctypes.data_as(C.POINTER(C.c_uint32)), _p(w, _f32p)))
        return out, ids, w

    def time_ms(self, batch: int, repeats: int = 20) -> float:
        ms = C.c_float(0)
        _check(load_library().quintrit_b200_moe_time(self._h, batch, repeats, C.byref(ms)))
        return ms.value

    def free(self) -> None:
        if self._h:
            load_library().quintrit_b200_moe_free(self._h)
            self._h = C.c_void_p()
        for m in self.matrices:
            m.free()
        self.matrices = []

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def sample_logits(logits, temperature: float, top_k: int, top_p: float, state: int, device: int = 0):
    """One draw of the device sampler from host logits: returns (token id, new generator state)."""
    lg = np.ascontiguousarray(logits, dtype=np.float32).reshape(-1)
    st, tok = C.c_uint64(state), C.c_uint32(0)
    lib = load_library()
    lib.quintrit_b200_sample_logits.argtypes = [C.c_uint32, _f32p, _sz, C.c_float, C.c_uint32, C.c_float, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)]
    _check(lib.quintrit_b200_sample_logits(device, _p(lg, _f32p), lg.size, temperature, top_k, top_p, C.byref(st), C.byref(tok)))
    return tok.value, st.value


def quantize_q8_0(x, device: int = 0):
    """Q8_0 activation blocks computed on the device: (codes int8[n], scales f32[n / 32])."""
    xx = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    q, d = np.zeros(xx.size, np.int8), np.zeros(xx.size // 32, np.float32)
    _check(load_library().quintrit_b200_quantize_q8_0(device, _p(xx, _f32p), xx.size, _p(q, _i8p), _p(d, _f32p)))
    return q, d


def gguf_describe(path: str) -> dict:
    """Hyperparameters and tensor directory of a GGUF file as the library reads them (host only, no GPU)."""
    n = _sz(0)
    lib = load_library()
    rc = lib.quintrit_b200_gguf_describe(str(path).encode(), None, 0, C.byref(n))
    if rc != 4:  # QUINTRIT_ERR_BUFFER_TOO_SMALL carries the size; anything else is the real outcome
        _check(rc)
    buf = C.create_string_buffer(n.value)
    _check(lib.quintrit_b200_gguf_describe(str(path).encode(), buf, n.value, C.byref(n)))
    out, tensors = {}, []
    for line in buf.value.decode().splitlines():
        key, _, rest = line.partition(" ")
        if key == "tensor":
            name, *fields = rest.split(" ")
            t = {"name": name, "inside_file": "outside-file" not in fields}
            for f in fields:
                if "=" in f:
                    k, v = f.split("=")
                    t[k] = tuple(int(x) for x in v.split("x")) if k == "shape" else int(v)
            tensors.append(t)
        else:
            out[key] = rest
    out["tensors"] = tensors
    return out
