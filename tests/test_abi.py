"""The C-ABI library loads without a GPU, exports every symbol the header declares, and validates arguments."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import quintrit_b200 as q

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(quintrit_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = q.load_library()
    names = _declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/ but not exported"


def test_versions_and_status_strings():
    lib = q.load_library()
    assert q.version().count(".") == 2
    assert lib.quintrit_b200_abi_version() == 1
    assert lib.quintrit_status_string(0) == b"success"
    assert lib.quintrit_status_string(15) == b"device error"
    assert lib.quintrit_status_string(99) == b"unknown status"


def test_null_pointers_and_struct_size_are_rejected():
    lib = q.load_library()
    assert lib.quintrit_cuda_device_count(None) == 1  # QUINTRIT_ERR_NULL_POINTER
    assert lib.quintrit_last_error_code() == 1
    assert b"NULL" in lib.quintrit_last_error_message()
    assert lib.quintrit_cuda_device_info(0, None) == 1
    from quintrit_b200.api import _DeviceInfoC

    info = _DeviceInfoC()
    info.struct_size = 8  # too small
    assert lib.quintrit_cuda_device_info(0, C.byref(info)) == 2
    h = C.c_void_p(123)
    assert lib.quintrit_b200_matrix_upload(0, 0, None, 0, 1, 1, C.byref(h)) == 1
    assert h.value is None  # the handle is cleared on failure
    assert lib.quintrit_b200_matrix_upload(0, 0, None, 0, 1, 1, None) == 1
    assert lib.quintrit_b200_matrix_free(None) == 0  # NULL is allowed
    assert lib.quintrit_b200_plan_free(None) == 0
    assert lib.quintrit_last_error_code() == 0 and lib.quintrit_last_error_message() == b""


def test_invalid_handles_shapes_and_sources():
    lib = q.load_library()
    junk = (C.c_uint8 * 256)()
    assert lib.quintrit_b200_matrix_info(C.cast(junk, C.c_void_p), None, None, None) == 14
    assert lib.quintrit_b200_gemv_i32(C.cast(junk, C.c_void_p), None, 0, None, 0) == 14
    assert lib.quintrit_b200_plan_launch(C.cast(junk, C.c_void_p), None) == 14
    data = np.zeros(64, np.uint8)
    h = C.c_void_p()
    p = data.ctypes.data_as(C.POINTER(C.c_uint8))
    assert lib.quintrit_b200_matrix_upload(0, 0, p, 64, 0, 160, C.byref(h)) == 3
    assert lib.quintrit_b200_matrix_upload(0, 0, p, 64, 1, 200000, C.byref(h)) == 3
    assert lib.quintrit_b200_matrix_upload(0, 7, p, 64, 1, 160, C.byref(h)) == 2
    assert lib.quintrit_b200_matrix_upload(0, 36, p, 64, 1, 160, C.byref(h)) == 8  # I2_S rows are multiples of 128
    assert lib.quintrit_b200_matrix_upload(0, 0, p, 16, 1, 160, C.byref(h)) == 4
    assert h.value is None


def test_pack_planar_matches_the_oracle_and_rejects_bad_trits(oracle):
    rng = np.random.default_rng(1)
    for rows, cols in [(1, 1), (3, 160), (4, 161), (5, 3072), (2, 319)]:
        t = rng.integers(-1, 2, rows * cols).astype(np.int8)
        assert np.array_equal(q.pack_planar(t, rows, cols), oracle.pack_planar(t, rows, cols))
    assert q.row_bytes(3072) == 640 and q.row_bytes(161) == 64
    bad = np.array([0, 2, 0], np.int8)
    with pytest.raises(q.QuintritError) as e:
        q.pack_planar(bad, 1, 3)
    assert e.value.code == 5


def test_device_count_never_fails():
    assert q.device_count() >= 0


def test_header_is_plain_c99_and_a_c_program_links(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 on its own, and a C program that calls into the library must
    link against it (no C++ or CUDA types in the signatures)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = os.path.join(root, "include", "quintrit_b200.h")
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-x", "c", header], check=True)
    src = tmp_path / "caller.c"
    src.write_text(
        '#include "quintrit_b200.h"\n#include <stdio.h>\n'
        "int main(void) {\n"
        "    uint32_t n = 0;\n"
        "    quintrit_gpu_options_t o = {sizeof o, 0, 0, 0};\n"
        "    quintrit_b200_decoder_t* d = NULL;\n"
        "    int rc = quintrit_cuda_device_count(&n);\n"
        '    if (quintrit_b200_decoder_open_gguf("no-such-file.gguf", &o, &d) != QUINTRIT_ERR_IO || d != NULL) return 2;\n'
        "    if (quintrit_b200_planar_row_bytes(3072) != 640) return 3;\n"
        '    printf("%s %u %d\\n", quintrit_b200_version(), (unsigned)n, rc);\n'
        "    return 0;\n}\n")
    exe = tmp_path / "caller"
    libdir = os.path.dirname(q.library_path())
    subprocess.run([gcc, "-std=c99", "-I", os.path.join(root, "include"), str(src), "-o", str(exe), "-L", libdir, "-lquintrit_b200",
                    f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True)
    assert out.stdout.split()[0] == q.version()
