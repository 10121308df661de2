"""What of the reference's C API can be checked without a GPU: the library exports every function of the reference's header,
programs written against that header compile and link against it unchanged, the format level reads the reference's own test
file, the oracle's decoders agree with the reference's packers, and handles and arguments are checked as the reference checks
them (rust/crates/quintrit-c/src/util.rs:10-183, runtime.rs:162-220)."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

import oracle
import quintrit_b200 as q
from oracle import gguf_model
from quintrit_b200.api import QuintritError
from quintrit_b200.runtime import GgufFile, _GenerateParams, _lib, _ModelInfo, _TensorInfo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
TINY = os.path.join(GOLDEN, "ref_tiny_model.gguf")
REFERENCE = os.environ.get("QUINTRIT_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))  # beside this repository, if anywhere
REF_HEADER = os.path.join(REFERENCE, "rust", "crates", "quintrit-c", "include", "quintrit.h")
needs_reference = pytest.mark.skipif(not os.path.exists(REF_HEADER), reason="the reference tree is not on this machine")

# the 45 functions of quintrit.h (ABI version 1), by level; kept here so that the check also runs where the reference is absent
REFERENCE_FUNCTIONS = """
quintrit_status_string quintrit_last_error_code quintrit_last_error_message quintrit_version quintrit_abi_version quintrit_cpu_features
quintrit_kernel_supported quintrit_kernel_resolve quintrit_kernel_name quintrit_kernel_tile_rows quintrit_supported_kernels quintrit_default_threads
quintrit_tiled_layout quintrit_tiled_size quintrit_pack_matrix quintrit_unpack_matrix quintrit_gemv_i32 quintrit_gemv_f32
quintrit_gguf_open quintrit_gguf_close quintrit_gguf_info quintrit_gguf_tensor_at quintrit_gguf_tensor_find quintrit_gguf_metadata_string
quintrit_gguf_metadata_u64 quintrit_gguf_tensor_data quintrit_gguf_tensor_layout quintrit_gguf_convert_tensor
quintrit_model_open quintrit_model_free quintrit_model_info quintrit_model_set_threads quintrit_model_tokenize quintrit_model_detokenize
quintrit_model_format_chat quintrit_session_create quintrit_session_free quintrit_session_reset quintrit_session_info
quintrit_generate_params_default quintrit_session_generate
quintrit_cuda_device_count quintrit_cuda_device_info quintrit_model_open_gpu quintrit_model_device
""".split()


def _exported():
    out = subprocess.run(["nm", "-D", "--defined-only", q.library_path()], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


def test_every_function_of_the_reference_header_is_exported():
    q.load_library()
    exported = _exported()
    assert len(REFERENCE_FUNCTIONS) == 45 and not [f for f in REFERENCE_FUNCTIONS if f not in exported]
    for extra in ("quintrit_session_feed_tokens", "quintrit_session_logits", "quintrit_session_generate_tokens"):
        assert extra in exported


@needs_reference
def test_the_list_above_is_the_reference_header():
    text = re.sub(r"/\*.*?\*/", "", open(REF_HEADER).read(), flags=re.S)
    declared = set(re.findall(r"QUINTRIT_API[^;(]*?\b(quintrit_[a-z0-9_]+)\s*\(", text))
    assert declared == set(REFERENCE_FUNCTIONS)


def _cc(tmp_path, source, name, include, std="c99", extra=()):
    lib_dir = os.path.dirname(q.library_path())
    exe = tmp_path / name
    r = subprocess.run(["gcc", f"-std={std}", "-Wall", "-Wextra", *extra, "-I", include, "-o", str(exe), source, "-L", lib_dir, "-lquintrit_b200", f"-Wl,-rpath,{lib_dir}"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


@needs_reference
@pytest.mark.parametrize("source", ["rust/crates/quintrit-c/tests/c/test_runtime.c", "rust/crates/quintrit-c/tests/c/test_kernel.c", "examples/c/generate_gpu.c",
                                    "examples/c/generate.c", "examples/c/gemv.c"])
def test_reference_c_programs_link_unchanged(tmp_path, source):
    q.load_library()
    exe = _cc(tmp_path, os.path.join(REFERENCE, source), "prog", os.path.dirname(REF_HEADER))
    r = subprocess.run([str(exe)], capture_output=True, text=True)  # without arguments each prints its usage (or runs host-only checks)
    assert r.returncode in (0, 1, 2)


@needs_reference
def test_struct_layouts_equal_the_reference_header(tmp_path):
    q.load_library()
    names = ["quintrit_tiled_layout_t", "quintrit_gguf_info_t", "quintrit_tensor_info_t", "quintrit_model_options_t", "quintrit_model_info_t", "quintrit_session_options_t",
             "quintrit_session_info_t", "quintrit_generate_params_t", "quintrit_generate_result_t", "quintrit_chat_message_t", "quintrit_cuda_device_info_t",
             "quintrit_gpu_options_t"]
    fields = ["offsetof(quintrit_model_info_t, architecture)", "offsetof(quintrit_tensor_info_t, name)", "offsetof(quintrit_generate_params_t, stop_sequences)",
              "offsetof(quintrit_cuda_device_info_t, name)", "offsetof(quintrit_tiled_layout_t, total_bytes)"]
    body = "".join(f'printf("%zu\\n", sizeof({n}));' for n in names) + "".join(f'printf("%zu\\n", {f});' for f in fields)
    outs = []
    for header, include in (("quintrit.h", os.path.dirname(REF_HEADER)), ("quintrit_b200_runtime.h", os.path.join(ROOT, "include"))):
        src = tmp_path / f"sizes_{header}.c"
        src.write_text(f'#include "{header}"\n#include <stddef.h>\n#include <stdio.h>\nint main(void) {{ {body} return 0; }}\n')
        outs.append(subprocess.run([str(_cc(tmp_path, str(src), "sizes", include))], capture_output=True, text=True, check=True).stdout)
    assert outs[0] == outs[1] and len(outs[0].split()) == len(names) + len(fields)
    # both headers in one translation unit, the reference's first
    both = tmp_path / "both.c"
    both.write_text('#include "quintrit.h"\n#include "quintrit_b200_runtime.h"\nint main(void) { return quintrit_abi_version() == QUINTRIT_ABI_VERSION && QUINTRIT_KERNEL_B200 == 16 ? 0 : 1; }\n')
    exe = _cc(tmp_path, str(both), "both", os.path.dirname(REF_HEADER), extra=("-I", os.path.join(ROOT, "include")))
    assert subprocess.run([str(exe)]).returncode == 0


def test_own_header_is_strict_c99_and_cxx(tmp_path):
    q.load_library()
    _cc(tmp_path, os.path.join(ROOT, "tests", "c", "runtime_acceptance.c"), "acc", os.path.join(ROOT, "include"), extra=("-pedantic", "-Werror"))
    src = tmp_path / "hdr.cpp"
    src.write_text('#include "quintrit_b200_runtime.h"\nint main() { return quintrit_abi_version() == 1 ? 0 : 1; }\n')
    lib_dir = os.path.dirname(q.library_path())
    r = subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), "-o", str(tmp_path / "hdr"), str(src), "-L", lib_dir,
                        "-lquintrit_b200", f"-Wl,-rpath,{lib_dir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert subprocess.run([str(tmp_path / "hdr")]).returncode == 0


def test_oracle_decoders_against_the_reference_packers():
    z = np.load(os.path.join(GOLDEN, "ref_builder_payloads.npz"))
    assert np.array_equal(oracle.decode_i2_s(z["i2s_payload"][:-4], 96, 256), z["i2s_trits"])
    assert np.frombuffer(z["i2s_payload"][-4:].tobytes(), np.float32)[0] == np.float32(0.125)
    assert np.array_equal(oracle.decode_tq2_0(z["tq2_payload"], 4, 256), z["tq2_trits"])
    assert oracle.uniform_block_scale(35, z["tq2_payload"]) == 0.5
    assert np.array_equal(oracle.encode_i2_s(z["i2s_trits"], 96, 256), z["i2s_payload"][:-4])


def test_format_level_on_the_reference_tiny_model():
    _, meta, tensors, data = gguf_model.read_gguf(TINY)
    with GgufFile(TINY) as f:
        assert f.version == 3 and len(f) == 21 == len(tensors) and f.n_metadata == len(meta) and f.data_start % 32 == 0
        infos = f.tensors()
        assert [t["name"] for t in infos] == list(tensors)  # file order
        for t in infos:
            shape, ty, off = tensors[t["name"]]
            assert t["ggml_shape"] == shape and t["dtype_id"] == ty and t["offset"] == off and t["is_ternary"] == (ty == 36)
            assert f.read_raw(t["name"]) == gguf_model.tensor_bytes(tensors, data, t["name"]).tobytes()
        t = f.tensor("blk.1.attn_k.weight")
        assert t["shape"] == [64, 128] and t["dtype"] == "I2_S" and t["n_elements"] == 64 * 128 and t["nbytes"] == 64 * 128 // 4
        assert f.tensor("token_embd.weight")["dtype"] == "F16" and f.tensor("output_norm.weight")["dtype"] == "F32"
        assert f.metadata_string("general.architecture") == "llama" and f.metadata_string("general.name") == "tiny-test-model"
        assert f.metadata_u64("llama.context_length") == 64 and f.metadata_u64("tokenizer.ggml.bos_token_id") == 259
        for call, code in ((lambda: f.tensor("missing"), 9), (lambda: f.metadata_string("nope"), 9), (lambda: f.metadata_string("llama.context_length"), 2),
                           (lambda: f.metadata_u64("general.name"), 2), (lambda: f.tensor_layout("token_embd.weight"), 8), (lambda: f.tensor_layout("blk.0.attn_q.weight", 2), 6),
                           (lambda: f.tensor_layout("blk.0.attn_q.weight", 77), 2)):
            with pytest.raises(QuintritError) as e:
                call()
            assert e.value.code == code
        lay, scale = f.tensor_layout("blk.0.ffn_gate.weight")
        assert (lay.kernel, lay.tile_rows, lay.rows, lay.cols, lay.padded_rows, lay.bytes_per_row, lay.total_bytes) == (16, 1, 256, 128, 256, 32, 256 * 32)
        assert scale == np.float32(0.05)
    with pytest.raises(QuintritError) as e:
        GgufFile(os.path.join(GOLDEN, "no-such.gguf"))
    assert e.value.code == 7
    with pytest.raises(QuintritError) as e:
        GgufFile(os.path.join(GOLDEN, "golden.npz"))
    assert e.value.code == 8


def test_kernel_level_queries_and_host_packing():
    l = _lib()
    out = C.c_int32(-1)
    assert l.quintrit_kernel_resolve(0, C.byref(out)) == 0 and out.value == 16
    assert l.quintrit_kernel_resolve(2, C.byref(out)) == 0 and out.value == 2
    assert l.quintrit_kernel_resolve(1234, C.byref(out)) == 2 and l.quintrit_kernel_supported(1234, C.byref(out)) == 2
    assert l.quintrit_kernel_supported(16, C.byref(out)) == 0 and out.value in (0, 1)
    assert [l.quintrit_kernel_name(k) for k in (0, 1, 2, 3, 16, 5)] == [b"auto", b"scalar", b"simd32", b"avx512", b"b200", None]
    n = C.c_size_t(0)
    assert l.quintrit_supported_kernels(None, 0, C.byref(n)) == 4 and n.value == 1
    ks = (C.c_int32 * 4)()
    assert l.quintrit_supported_kernels(ks, 4, C.byref(n)) == 0 and ks[0] == 16
    assert l.quintrit_kernel_tile_rows(0, C.byref(n)) == 0 and n.value == 1 and l.quintrit_kernel_tile_rows(3, C.byref(n)) == 6
    assert l.quintrit_tiled_size(0, 100, 1000, C.byref(n)) == 0 and n.value == 100 * 7 * 32
    assert l.quintrit_tiled_size(0, 0, 1000, C.byref(n)) == 3
    th = C.c_uint32(0)
    assert l.quintrit_default_threads(C.byref(th)) == 0 and 1 <= th.value <= 256
    mask = C.c_uint64(0)
    assert l.quintrit_cpu_features(C.byref(mask)) == 0 and l.quintrit_cpu_features(None) == 1
    # pack and unpack on the host round-trip, for a column count with a ragged tail
    rng = np.random.default_rng(5)
    trits = rng.integers(-1, 2, size=(7, 333)).astype(np.int8)
    packed = np.zeros(7 * 3 * 32, np.uint8)
    i8p, u8p = C.POINTER(C.c_int8), C.POINTER(C.c_uint8)
    l.quintrit_pack_matrix.argtypes = [C.c_int32, i8p, C.c_size_t, C.c_size_t, C.c_size_t, u8p, C.c_size_t]
    l.quintrit_unpack_matrix.argtypes = [C.c_int32, u8p, C.c_size_t, C.c_size_t, C.c_size_t, i8p, C.c_size_t]
    assert l.quintrit_pack_matrix(0, trits.ctypes.data_as(i8p), trits.size, 7, 333, packed.ctypes.data_as(u8p), packed.size) == 0
    assert np.array_equal(packed, oracle.pack_planar(trits, 7, 333).reshape(-1))
    back = np.full((7, 333), 9, np.int8)
    assert l.quintrit_unpack_matrix(16, packed.ctypes.data_as(u8p), packed.size, 7, 333, back.ctypes.data_as(i8p), back.size) == 0
    assert np.array_equal(back, trits)
    assert l.quintrit_unpack_matrix(16, packed.ctypes.data_as(u8p), packed.size - 1, 7, 333, back.ctypes.data_as(i8p), back.size) == 4
    packed[5] = 251  # not a velurex code
    assert l.quintrit_unpack_matrix(16, packed.ctypes.data_as(u8p), packed.size, 7, 333, back.ctypes.data_as(i8p), back.size) == 5
    assert l.quintrit_pack_matrix(2, trits.ctypes.data_as(i8p), trits.size, 7, 333, packed.ctypes.data_as(u8p), packed.size) == 6  # a CPU kernel's layout


def test_handles_and_arguments_are_checked_without_a_device():
    l = _lib()
    assert l.quintrit_version() == b"0.2.0" and l.quintrit_abi_version() == 1
    assert l.quintrit_model_free(None) == 0 and l.quintrit_session_free(None) == 0 and l.quintrit_gguf_close(None) == 0
    info = _ModelInfo(struct_size=C.sizeof(_ModelInfo))
    assert l.quintrit_model_info(None, C.byref(info)) == 14
    junk = C.create_string_buffer(64)  # a pointer to something that is not a handle
    assert l.quintrit_model_info(junk, C.byref(info)) == 14 and l.quintrit_session_reset(junk) == 14 and l.quintrit_gguf_close(junk) == 14
    ti = _TensorInfo(struct_size=C.sizeof(_TensorInfo))
    assert l.quintrit_gguf_tensor_at(None, 0, C.byref(ti)) == 14
    h = C.c_void_p(1)
    assert l.quintrit_model_open_gpu(b"no-such-file.gguf", None, C.byref(h)) == 7 and h.value is None
    assert l.quintrit_model_open(b"no-such-file.gguf", None, C.byref(h)) == 7 and h.value is None
    assert l.quintrit_model_open_gpu(None, None, C.byref(h)) == 1 and l.quintrit_model_open_gpu(b"x", None, None) == 1
    assert l.quintrit_model_open_gpu(os.path.join(GOLDEN, "golden.npz").encode(), None, C.byref(h)) == 8
    p = _GenerateParams()
    assert l.quintrit_generate_params_default(C.byref(p)) == 0 and l.quintrit_generate_params_default(None) == 1
    assert (p.struct_size, p.flags, p.max_tokens, p.top_k, p.temperature, p.top_p, p.seed, p.stop_count) == (C.sizeof(_GenerateParams), 0, 128, 1, 0.0, 1.0, 0, 0)
    assert l.quintrit_session_feed_tokens(None, None, 0, 0) == 14 and b"handle" in l.quintrit_last_error_message()
