"""Builds the CUDA library in-tree with nvcc for sm_100a.

``python -m humming_b200.build`` compiles ``csrc/api.cu`` (which includes every
kernel) into ``humming_b200/lib/libhumming_b200.so``.  nvcc cross-compiles, so
this works on a machine without a GPU.
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(PKG_DIR, "csrc", "api.cu")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libhumming_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def find_nvcc():
    for cand in (os.environ.get("CUDA_NVCC_PATH"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set CUDA_NVCC_PATH)")


def sources():
    csrc = os.path.join(PKG_DIR, "csrc")
    inc = os.path.join(os.path.dirname(PKG_DIR), "include")
    out = [os.path.join(csrc, f) for f in sorted(os.listdir(csrc))]
    out += [os.path.join(inc, f) for f in sorted(os.listdir(inc))]
    return out


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > t for s in sources())


def build(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    extra = os.environ.get("HM_NVCC_EXTRA", "").split()  # e.g. -DNAME=value switches while developing kernels
    cmd = [find_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH, SRC]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libhumming_b200.so")
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
