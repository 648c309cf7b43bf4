"""Builds the CUDA library of kernl_b200 in-tree with nvcc for sm_100a.

`python -m kernl_b200.build` writes kernl_b200/libkernl_b200.so next to this file. nvcc
cross-compiles without a GPU, so this runs on any box that has the CUDA toolkit.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libkernl_b200.so")
SOURCES = ["kernl_b200.cu"]
HEADERS = ["common.cuh", "norm.cuh", "linear.cuh", "linear_pair.cuh", "linear_smallm.cuh", "attention.cuh", "attention_split.cuh", "attention_persist.cuh", "attention_decode.cuh", "allreduce.cuh", "rope.cuh"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--shared",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the kernl_b200 CUDA library cannot be built")
    return exe


HASH_PATH = LIB_PATH + ".srchash"


def _source_hash() -> str:
    """Hash of everything the library is built from (sources, headers, flags)."""
    import hashlib

    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    deps += [os.path.join(HERE, "..", "include", "kernl_b200.h"), os.path.join(HERE, "..", "include", "kernl_b200_debug.h")]
    for d in deps:
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def is_stale() -> bool:
    """The library is rebuilt when it is missing or was built from other sources. By content, not by
    modification time: a copy of the tree to another machine keeps the contents, not the times."""
    if not os.path.exists(LIB_PATH) or not os.path.exists(HASH_PATH):
        return True
    try:
        return open(HASH_PATH).read().strip() != _source_hash()
    except OSError:
        return True


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/*.cu into libkernl_b200.so (skipped when up to date). Returns the path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    with open(HASH_PATH, "w") as f:
        f.write(_source_hash() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
