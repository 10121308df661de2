"""Builds libquintrit_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import fcntl
import hashlib
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libquintrit_b200.so")
SOURCES = ["csrc/capi.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


STAMP = LIB + ".srchash"  # hash of the sources the library was built from (file times do not survive every copy of the tree)


def _source_files():
    srcs = [os.path.join(HERE, "csrc", f) for f in sorted(os.listdir(os.path.join(HERE, "csrc"))) if f.endswith((".cu", ".cuh", ".hpp", ".h"))]
    inc = os.path.join(os.path.dirname(HERE), "include")
    return srcs + [os.path.join(inc, f) for f in sorted(os.listdir(inc)) if f.endswith(".h")]


def _source_hash() -> str:
    h = hashlib.sha256()
    for path in _source_files():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + os.environ.get("QUINTRIT_B200_NVCC_EXTRA", "").split()).encode())
    return h.hexdigest()


def needs_build() -> bool:
    if not os.path.exists(LIB) or not os.path.exists(STAMP):
        return True
    try:
        return open(STAMP).read().strip() != _source_hash()
    except OSError:
        return True


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library if its sources changed. Safe to call from several processes at once (one rank per GPU): a file lock lets one of
    them compile into a temporary file that is renamed into place; the others find the library up to date when they get the lock."""
    if not force and not needs_build():
        return LIB
    with open(os.path.join(HERE, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if force or needs_build():
                extra = os.environ.get("QUINTRIT_B200_NVCC_EXTRA", "").split()  # experiment knob, e.g. -DQTB_GEMV_DEPTH=2
                tmp = f"{LIB}.tmp.{os.getpid()}"
                cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-o", tmp, *[os.path.join(HERE, s) for s in SOURCES]]
                if verbose:
                    cmd.insert(1, "-Xptxas")
                    cmd.insert(2, "-v")
                r = subprocess.run(cmd, capture_output=True, text=True)
                if r.returncode != 0:
                    if os.path.exists(tmp):
                        os.remove(tmp)
                    raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
                os.replace(tmp, LIB)
                with open(STAMP + ".tmp", "w") as f:
                    f.write(_source_hash())
                os.replace(STAMP + ".tmp", STAMP)
                if verbose:
                    print(r.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))
