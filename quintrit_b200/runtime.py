"""Python host side of the runtime level: ``Model``, ``Tokenizer``, ``GgufFile`` over the reference's C API as
``libquintrit_b200.so`` exports it (quintrit_model_open_gpu, quintrit_session_generate, ... - see
``include/quintrit_b200_runtime.h``).

The class and method names, defaults and argument meaning follow the reference's Python binding
(rust/crates/quintrit-py/src/runtime.rs:540-800: ``Model.load(path, device=, context=)``, ``generate``, ``stream``,
``chat``, ``format_chat``, ``logits``, ``tokenizer.encode / decode / decode_pieces``) so that tests written against it read
the same here. Every call goes through the C ABI; there is no CPU path (``device`` must name a CUDA device).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from .api import QuintritError, _check, load_library

_sz = C.c_size_t
FINISH = {0: "length", 1: "eos", 2: "stop", 3: "callback", 4: "context"}


class _GpuOptions(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("device_index", C.c_uint32), ("context_length", C.c_uint32), ("flags", C.c_uint32)]


class _ModelInfo(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("kernel", C.c_int32), ("num_threads", C.c_uint32), ("num_layers", C.c_uint32), ("hidden_size", C.c_uint32),
                ("num_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("vocab_size", C.c_uint64), ("context_length", C.c_uint64),
                ("bos_token_id", C.c_int64), ("eos_token_id", C.c_int64), ("architecture", C.c_char * 16)]


class _SessionOptions(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("context_length", C.c_uint32)]


class _SessionInfo(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("reserved", C.c_uint32), ("context_length", C.c_uint64), ("position", C.c_uint64)]


class _GenerateParams(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("flags", C.c_uint32), ("max_tokens", C.c_uint32), ("top_k", C.c_uint32), ("temperature", C.c_float),
                ("top_p", C.c_float), ("seed", C.c_uint64), ("stop_sequences", C.POINTER(C.c_char_p)), ("stop_count", _sz)]


class _GenerateResult(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("finish_reason", C.c_int32), ("prompt_tokens", C.c_uint32), ("generated_tokens", C.c_uint32),
                ("text_bytes", C.c_uint64)]


class _ChatMessage(C.Structure):
    _fields_ = [("role", C.c_char_p), ("content", C.c_char_p)]


class _GgufInfo(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("version", C.c_uint32), ("tensor_count", C.c_uint64), ("metadata_count", C.c_uint64), ("data_offset", C.c_uint64)]


class _TensorInfo(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("ggml_type", C.c_int32), ("n_dims", C.c_uint32), ("is_ternary", C.c_int32), ("shape", C.c_uint64 * 8),
                ("num_elements", C.c_uint64), ("offset", C.c_uint64), ("data_bytes", C.c_uint64), ("name", C.c_char_p), ("type_name", C.c_char_p)]


class _TiledLayout(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("kernel", C.c_int32), ("tile_rows", C.c_uint64), ("rows", C.c_uint64), ("cols", C.c_uint64),
                ("padded_rows", C.c_uint64), ("bytes_per_row", C.c_uint64), ("total_bytes", C.c_uint64)]


TOKEN_CALLBACK = C.CFUNCTYPE(C.c_int, C.POINTER(C.c_char), _sz, C.c_void_p)
_declared = False


def _lib() -> C.CDLL:
    global _declared
    l = load_library()
    if _declared:
        return l
    vp, u32p = C.c_void_p, C.POINTER(C.c_uint32)
    l.quintrit_version.restype = C.c_char_p
    l.quintrit_abi_version.restype = C.c_uint32
    l.quintrit_kernel_name.restype = C.c_char_p
    l.quintrit_kernel_name.argtypes = [C.c_int32]
    l.quintrit_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    l.quintrit_gguf_close.argtypes = [vp]
    l.quintrit_gguf_info.argtypes = [vp, C.POINTER(_GgufInfo)]
    l.quintrit_gguf_tensor_at.argtypes = [vp, _sz, C.POINTER(_TensorInfo)]
    l.quintrit_gguf_tensor_find.argtypes = [vp, C.c_char_p, C.POINTER(_TensorInfo)]
    l.quintrit_gguf_metadata_string.argtypes = [vp, C.c_char_p, C.c_char_p, _sz, C.POINTER(_sz)]
    l.quintrit_gguf_metadata_u64.argtypes = [vp, C.c_char_p, C.POINTER(C.c_uint64)]
    l.quintrit_gguf_tensor_data.argtypes = [vp, C.c_char_p, C.POINTER(C.POINTER(C.c_uint8)), C.POINTER(_sz)]
    l.quintrit_gguf_tensor_layout.argtypes = [vp, C.c_char_p, C.c_int32, C.POINTER(_TiledLayout), C.POINTER(C.c_float)]
    l.quintrit_gguf_convert_tensor.argtypes = [vp, C.c_char_p, C.c_int32, C.POINTER(C.c_uint8), _sz, C.POINTER(_TiledLayout), C.POINTER(C.c_float)]
    l.quintrit_model_open_gpu.argtypes = [C.c_char_p, C.POINTER(_GpuOptions), C.POINTER(vp)]
    l.quintrit_model_open.argtypes = [C.c_char_p, vp, C.POINTER(vp)]
    l.quintrit_model_free.argtypes = [vp]
    l.quintrit_model_info.argtypes = [vp, C.POINTER(_ModelInfo)]
    l.quintrit_model_set_threads.argtypes = [vp, C.c_uint32]
    l.quintrit_model_device.argtypes = [vp, C.POINTER(C.c_int32), u32p]
    l.quintrit_model_tokenize.argtypes = [vp, C.c_char_p, _sz, C.c_uint32, u32p, _sz, C.POINTER(_sz)]
    l.quintrit_model_detokenize.argtypes = [vp, u32p, _sz, C.c_char_p, _sz, C.POINTER(_sz)]
    l.quintrit_model_format_chat.argtypes = [vp, C.POINTER(_ChatMessage), _sz, C.c_char_p, _sz, C.POINTER(_sz)]
    l.quintrit_session_create.argtypes = [vp, C.POINTER(_SessionOptions), C.POINTER(vp)]
    l.quintrit_session_free.argtypes = [vp]
    l.quintrit_session_reset.argtypes = [vp]
    l.quintrit_session_info.argtypes = [vp, C.POINTER(_SessionInfo)]
    l.quintrit_generate_params_default.argtypes = [C.POINTER(_GenerateParams)]
    l.quintrit_session_generate.argtypes = [vp, C.c_char_p, _sz, C.POINTER(_GenerateParams), TOKEN_CALLBACK, vp, C.c_char_p, _sz, C.POINTER(_sz),
                                            C.POINTER(_GenerateResult)]
    l.quintrit_session_feed_tokens.argtypes = [vp, u32p, _sz, C.c_uint32]
    l.quintrit_session_logits.argtypes = [vp, C.POINTER(C.c_float), _sz]
    l.quintrit_session_generate_tokens.argtypes = [vp, u32p, _sz, _sz, u32p, _sz, C.POINTER(_sz)]
    l.quintrit_b200_tokenizer_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    l.quintrit_b200_tokenizer_free.argtypes = [vp]
    l.quintrit_b200_tokenizer_info.argtypes = [vp, C.POINTER(C.c_uint64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    l.quintrit_b200_tokenizer_encode.argtypes = [vp, C.c_char_p, _sz, C.c_uint32, u32p, _sz, C.POINTER(_sz)]
    l.quintrit_b200_tokenizer_decode.argtypes = [vp, u32p, _sz, C.c_int, C.c_char_p, _sz, C.POINTER(_sz), C.POINTER(_sz)]
    _declared = True
    return l


def _ids(tokens) -> np.ndarray:
    a = np.asarray(list(tokens), dtype=np.int64)
    if a.size and (a.min() < 0 or a.max() > 0xFFFFFFFF):
        raise OverflowError("token ids must fit an unsigned 32-bit integer")
    return np.ascontiguousarray(a.astype(np.uint32))


def _u32p(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_uint32))


def _sized_text(call) -> str:
    """Runs the size query / fill protocol of the C API (QUINTRIT_ERR_BUFFER_TOO_SMALL = 4 reports the needed length)."""
    n = _sz(0)
    rc = call(None, 0, C.byref(n))
    if rc not in (0, 4):
        _check(rc)
    buf = C.create_string_buffer(n.value + 1)
    _check(call(buf, n.value + 1, C.byref(n)))
    return buf.raw[:n.value].decode("utf-8")


class Tokenizer:
    """Byte-level BPE tokenizer of a GGUF file (quintrit-runtime/src/tokenizer.rs). Opened on its own it needs no GPU."""

    def __init__(self, path=None, *, _model=None):
        self._l = _lib()
        self._model = _model
        self._h = C.c_void_p()
        if _model is None:
            _check(self._l.quintrit_b200_tokenizer_open(os.fsencode(str(path)), C.byref(self._h)))
            v, b, e = C.c_uint64(), C.c_int64(), C.c_int64()
            _check(self._l.quintrit_b200_tokenizer_info(self._h, C.byref(v), C.byref(b), C.byref(e)))
            self.vocab_size, bos, eos = v.value, b.value, e.value
        else:
            self.vocab_size, bos, eos = _model.vocab_size, _model._info.bos_token_id, _model._info.eos_token_id
        self.bos_token_id = None if bos < 0 else bos
        self.eos_token_id = None if eos < 0 else eos

    def __len__(self) -> int:
        return self.vocab_size

    def encode(self, text: str, add_bos: bool = False) -> list[int]:
        if not isinstance(text, str):
            raise TypeError("text must be a str")
        raw = text.encode("utf-8")
        n = _sz(0)
        flags = 1 if add_bos else 0
        if self._model is not None:
            call = lambda out, cap: self._l.quintrit_model_tokenize(self._model._h, raw, len(raw), flags, out, cap, C.byref(n))  # noqa: E731
        else:
            call = lambda out, cap: self._l.quintrit_b200_tokenizer_encode(self._h, raw, len(raw), flags, out, cap, C.byref(n))  # noqa: E731
        rc = call(None, 0)
        if rc not in (0, 4):
            _check(rc)
        out = np.zeros(max(n.value, 1), np.uint32)
        _check(call(_u32p(out), out.size))
        return out[:n.value].tolist()

    def decode(self, tokens) -> str:
        if isinstance(tokens, (str, bytes)):
            raise TypeError("tokens must be a sequence of token ids")
        ids = _ids(tokens)
        if self._model is not None:
            return _sized_text(lambda buf, cap, n: self._l.quintrit_model_detokenize(self._model._h, _u32p(ids), ids.size, buf, cap, n))
        return _sized_text(lambda buf, cap, n: self._l.quintrit_b200_tokenizer_decode(self._h, _u32p(ids), ids.size, 0, buf, cap, n, None))

    def decode_token(self, token: int) -> str:
        return self.decode([token])

    def decode_pieces(self, tokens) -> list[str]:
        """The text piece every token adds when decoded as a stream, plus the final flush: characters are never split."""
        if self._h.value is None:
            raise QuintritError(6, "decode_pieces needs a Tokenizer opened from the file (Tokenizer(path))")
        ids = _ids(tokens)
        ends = (_sz * (ids.size + 1))()
        text = _sized_text(lambda buf, cap, n: self._l.quintrit_b200_tokenizer_decode(self._h, _u32p(ids), ids.size, 1, buf, cap, n, ends)).encode("utf-8")
        cuts = [0] + list(ends)
        return [text[a:b].decode("utf-8") for a, b in zip(cuts[:-1], cuts[1:])]

    def __del__(self):
        try:
            if self._h.value is not None:
                self._l.quintrit_b200_tokenizer_free(self._h)
        except Exception:
            pass


class TokenStream:
    """Result of ``Model.stream``: the pieces in the order the callback received them (the generation has finished)."""

    def __init__(self, pieces, reason, n_tokens, prompt_tokens):
        self._pieces = list(pieces)
        self.text = "".join(pieces)
        self.finish_reason, self.n_tokens, self.prompt_tokens = reason, n_tokens, prompt_tokens

    def __iter__(self):
        return self

    def __next__(self) -> str:
        if not self._pieces:
            raise StopIteration
        return self._pieces.pop(0)


class Model:
    """A model on a B200 with one session (quintrit_model_open_gpu + quintrit_session_create)."""

    def __init__(self, handle, lib, path):
        self._h, self._l, self.path = handle, lib, str(path)
        self._info = _ModelInfo(struct_size=C.sizeof(_ModelInfo))
        _check(lib.quintrit_model_info(handle, C.byref(self._info)))
        self._s = C.c_void_p()
        _check(lib.quintrit_session_create(handle, None, C.byref(self._s)))
        si = _SessionInfo(struct_size=C.sizeof(_SessionInfo))
        _check(lib.quintrit_session_info(self._s, C.byref(si)))
        self.context_window = si.context_length
        dev, idx = C.c_int32(), C.c_uint32()
        _check(lib.quintrit_model_device(handle, C.byref(dev), C.byref(idx)))
        self.device = f"cuda:{idx.value}" if dev.value == 1 else "cpu"
        self.tokenizer = Tokenizer(_model=self)

    @staticmethod
    def load(path, *, device: str = "cuda", context: int | None = None, verbose: bool = False) -> "Model":
        if device == "cuda":
            index = 0
        elif device.startswith("cuda:") and device[5:].isdigit():
            index = int(device[5:])
        else:
            raise QuintritError(2, f"device {device!r} is not 'cuda' or 'cuda:N' (this library has no CPU engine)")
        l = _lib()
        opts = _GpuOptions(struct_size=C.sizeof(_GpuOptions), device_index=index, context_length=context or 0, flags=1 if verbose else 0)
        h = C.c_void_p()
        _check(l.quintrit_model_open_gpu(os.fsencode(str(path)), C.byref(opts), C.byref(h)))
        return Model(h, l, path)

    architecture = property(lambda self: self._info.architecture.decode())
    vocab_size = property(lambda self: self._info.vocab_size)
    context_length = property(lambda self: self._info.context_length)
    n_layers = property(lambda self: self._info.num_layers)
    hidden_size = property(lambda self: self._info.hidden_size)
    threads = property(lambda self: self._info.num_threads)
    kernel = property(lambda self: "cuda")

    @property
    def config(self) -> dict:
        i = self._info
        return {"num_attention_heads": i.num_heads, "num_key_value_heads": i.num_kv_heads, "head_dim": i.head_dim, "hidden_size": i.hidden_size,
                "num_hidden_layers": i.num_layers, "bos_token_id": None if i.bos_token_id < 0 else i.bos_token_id,
                "eos_token_id": None if i.eos_token_id < 0 else i.eos_token_id}

    @property
    def position(self) -> int:
        si = _SessionInfo(struct_size=C.sizeof(_SessionInfo))
        _check(self._l.quintrit_session_info(self._s, C.byref(si)))
        return si.position

    def reset(self) -> None:
        _check(self._l.quintrit_session_reset(self._s))

    def _run(self, prompt: str, max_tokens: int, temperature: float, top_k: int, top_p: float, seed: int, stop, keep_context: bool, on_piece=None) -> TokenStream:
        if not isinstance(prompt, str):
            raise TypeError("prompt must be a str")
        if max_tokens < 0 or top_k < 0:
            raise ValueError("max_tokens and top_k must not be negative")
        p = _GenerateParams()
        _check(self._l.quintrit_generate_params_default(C.byref(p)))
        p.max_tokens, p.top_k, p.temperature, p.top_p, p.seed = max_tokens, top_k, temperature, top_p, seed
        p.flags = 1 if keep_context else 0
        stops = [stop] if isinstance(stop, str) else list(stop or [])
        raw_stops = [s.encode("utf-8") for s in stops]
        arr = (C.c_char_p * max(len(raw_stops), 1))(*raw_stops)
        if raw_stops:
            p.stop_sequences, p.stop_count = C.cast(arr, C.POINTER(C.c_char_p)), len(raw_stops)
        pieces: list[bytes] = []

        def cb(text, n, _user):
            piece = C.string_at(text, n)
            pieces.append(piece)
            return 1 if on_piece is not None and on_piece(piece.decode("utf-8")) else 0

        res = _GenerateResult(struct_size=C.sizeof(_GenerateResult))
        raw = prompt.encode("utf-8")
        cap = 64 + 64 * max_tokens
        out, n = C.create_string_buffer(cap), _sz(0)
        _check(self._l.quintrit_session_generate(self._s, raw, len(raw), C.byref(p), TOKEN_CALLBACK(cb), None, out, cap, C.byref(n), C.byref(res)))
        ts = TokenStream([b.decode("utf-8") for b in pieces], FINISH[res.finish_reason], res.generated_tokens, res.prompt_tokens)
        ts.buffer_text = out.raw[:min(n.value, cap - 1)].decode("utf-8", "replace")
        ts.text_bytes = res.text_bytes
        return ts

    def generate(self, prompt: str, max_tokens: int = 128, *, temperature: float = 0.0, top_k: int = 40, top_p: float = 0.9, seed: int = 42, stop=None,
                 keep_context: bool = False) -> str:
        return self._run(prompt, max_tokens, temperature, top_k, top_p, seed, stop, keep_context).buffer_text

    def stream(self, prompt: str, max_tokens: int = 128, *, temperature: float = 0.0, top_k: int = 40, top_p: float = 0.9, seed: int = 42, stop=None,
               on_piece=None) -> TokenStream:
        return self._run(prompt, max_tokens, temperature, top_k, top_p, seed, stop, False, on_piece)

    def format_chat(self, messages) -> str:
        msgs = (_ChatMessage * max(len(messages), 1))()
        keep = []
        for i, m in enumerate(messages):
            r, c = m["role"].encode("utf-8"), m["content"].encode("utf-8")
            keep += [r, c]
            msgs[i].role, msgs[i].content = r, c
        return _sized_text(lambda buf, cap, n: self._l.quintrit_model_format_chat(self._h, msgs, len(messages), buf, cap, n))

    def chat(self, messages, max_tokens: int = 128, **kw) -> str:
        return self.generate(self.format_chat(messages), max_tokens, **kw)

    def logits(self, prompt, keep_context: bool = False) -> np.ndarray:
        """Next-token logits after the prompt (text: BOS is put in front if the model has one; or a list of token ids)."""
        if isinstance(prompt, str):
            ids = self.tokenizer.encode(prompt, add_bos=True)
        else:
            ids = prompt
        a = _ids(ids)
        _check(self._l.quintrit_session_feed_tokens(self._s, _u32p(a), a.size, 1 if keep_context else 0))
        out = np.zeros(self.vocab_size, np.float32)
        _check(self._l.quintrit_session_logits(self._s, out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def reused_tokens(self) -> int:
        """Prompt tokens the last ``generate`` / ``stream`` call found in the KV cache and did not compute again."""
        n = C.c_uint32(0)
        _check(self._l.quintrit_b200_session_reused_tokens(self._s, C.byref(n)))
        return n.value

    def generate_tokens(self, prompt_ids, max_new: int) -> np.ndarray:
        a = _ids(prompt_ids)
        out, n = np.zeros(max_new, np.uint32), _sz(0)
        _check(self._l.quintrit_session_generate_tokens(self._s, _u32p(a), a.size, max_new, _u32p(out), out.size, C.byref(n)))
        return out[:n.value]

    def close(self) -> None:
        if self._s.value is not None:
            self._l.quintrit_session_free(self._s)
            self._s = C.c_void_p()
        if self._h.value is not None:
            self._l.quintrit_model_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __repr__(self) -> str:
        return f"Model({self.path!r}, architecture={self.architecture!r}, device={self.device!r})"


class GgufFile:
    """A GGUF file opened through the format level of the C API (quintrit_gguf_*); host only."""

    def __init__(self, path):
        self._l = _lib()
        self._h = C.c_void_p()
        self.path = str(path)
        _check(self._l.quintrit_gguf_open(os.fsencode(self.path), C.byref(self._h)))
        info = _GgufInfo(struct_size=C.sizeof(_GgufInfo))
        _check(self._l.quintrit_gguf_info(self._h, C.byref(info)))
        self.version, self.n_metadata, self.data_start, self._n = info.version, info.metadata_count, info.data_offset, info.tensor_count

    def __len__(self) -> int:
        return self._n

    @staticmethod
    def _tensor(t: _TensorInfo) -> dict:
        return {"name": t.name.decode(), "ggml_shape": list(t.shape[:t.n_dims]), "shape": list(t.shape[:t.n_dims])[::-1], "dtype": t.type_name.decode(),
                "dtype_id": t.ggml_type, "is_ternary": bool(t.is_ternary), "n_elements": t.num_elements, "nbytes": t.data_bytes, "offset": t.offset}

    def tensors(self) -> list[dict]:
        out = []
        for i in range(self._n):
            t = _TensorInfo(struct_size=C.sizeof(_TensorInfo))
            _check(self._l.quintrit_gguf_tensor_at(self._h, i, C.byref(t)))
            out.append(self._tensor(t))
        return out

    def tensor(self, name: str) -> dict:
        t = _TensorInfo(struct_size=C.sizeof(_TensorInfo))
        _check(self._l.quintrit_gguf_tensor_find(self._h, name.encode(), C.byref(t)))
        return self._tensor(t)

    def metadata_string(self, key: str) -> str:
        return _sized_text(lambda buf, cap, n: self._l.quintrit_gguf_metadata_string(self._h, key.encode(), buf, cap, n))

    def metadata_u64(self, key: str) -> int:
        v = C.c_uint64()
        _check(self._l.quintrit_gguf_metadata_u64(self._h, key.encode(), C.byref(v)))
        return v.value

    def read_raw(self, name: str) -> bytes:
        p, n = C.POINTER(C.c_uint8)(), _sz(0)
        _check(self._l.quintrit_gguf_tensor_data(self._h, name.encode(), C.byref(p), C.byref(n)))
        return C.string_at(p, n.value)

    def tensor_layout(self, name: str, kernel: int = 0):
        lay, scale = _TiledLayout(struct_size=C.sizeof(_TiledLayout)), C.c_float()
        _check(self._l.quintrit_gguf_tensor_layout(self._h, name.encode(), kernel, C.byref(lay), C.byref(scale)))
        return lay, scale.value

    def convert_tensor(self, name: str, kernel: int = 0):
        """(planar bytes, rows, cols, scale): the tensor transcoded on the GPU into the device kernel's host-visible layout."""
        lay, _ = self.tensor_layout(name, kernel)
        out, scale = np.zeros(lay.total_bytes, np.uint8), C.c_float()
        _check(self._l.quintrit_gguf_convert_tensor(self._h, name.encode(), lay.kernel, out.ctypes.data_as(C.POINTER(C.c_uint8)), out.size, C.byref(lay),
                                                    C.byref(scale)))
        return out, lay.rows, lay.cols, np.float32(scale.value)

    def close(self) -> None:
        if self._h.value is not None:
            _check(self._l.quintrit_gguf_close(self._h))
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
