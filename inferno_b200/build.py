"""In-tree build of the CUDA library: ``python -m inferno_b200.build``.

Compiles ``csrc/attn_api.cu`` (which includes every kernel) for sm_100a into
``inferno_b200/lib/libinferno_b200_attn.so``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libinferno_b200_attn.so")
# The checked build (-DIB200_BOUNDS): every TMA coordinate, tensor-memory address and swizzled shared-memory store is
# range-checked on the device; a violation is recorded in the status word and the access skipped.  Same ABI; select it
# with the environment variable IB200_LIB.  For debugging and for one pass of the small-shape parity tests.
BOUNDS_LIB_PATH = os.path.join(LIB_DIR, "libinferno_b200_attn_bounds.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "--use_fast_math", "-Xcompiler", "-fPIC", "-shared"]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh")))


def is_stale(path: str = LIB_PATH) -> bool:
    if not os.path.isfile(path):
        return True
    t = os.path.getmtime(path)
    hdr = os.path.join(os.path.dirname(HERE), "include", "inferno_b200_attn.h")
    return any(os.path.getmtime(s) > t for s in sources() + [hdr])


def build(force: bool = False, verbose: bool = False, bounds: bool = False) -> str:
    out = BOUNDS_LIB_PATH if bounds else LIB_PATH
    if not force and not is_stale(out):
        return out
    os.makedirs(LIB_DIR, exist_ok=True)
    extra = os.environ.get("IB200_NVCC_FLAGS", "").split()      # extra defines for tuning experiments
    if bounds:
        extra.append("-DIB200_BOUNDS=1")
    cmd = [NVCC] + FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-o", out, os.path.join(CSRC, "attn_api.cu")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building " + out)
    return out


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv, bounds="--bounds" in sys.argv))
