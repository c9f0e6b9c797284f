"""Build recipe of oracle/_ref/: the reference's own host check GEMM (a CUTLASS template), compiled on its own.

TEST / BASELINE INFRASTRUCTURE. The reference's `--reference-check` multiplies with
``cutlass::reference::host::Gemm`` (tests/kernel_test.cu:441-456 of the reference). CUTLASS is an un-vendored
git submodule there; this machine carries copies of its headers inside Python packages, and
``oracle/ref_host_gemm.cpp`` instantiates exactly the reference's template arguments against them. Host code
only (nvcc is used as the driver because the CUTLASS headers name CUDA intrinsics); no GPU is needed to build or
run it. Output goes to oracle/_ref/, which is not part of the source tree.

    python -m oracle.build_ref        # prints the path of the binary, or why it cannot be built
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
BINARY = os.path.join(OUT_DIR, "ref_host_gemm")
SOURCE = os.path.join(HERE, "ref_host_gemm.cpp")


def find_cutlass():
    """Root of a CUTLASS copy that has both the core headers and the host reference utilities."""
    roots = []
    for p in sys.path:
        roots += glob.glob(os.path.join(p, "flashinfer", "data", "cutlass")) + glob.glob(os.path.join(p, "tilelang", "3rdparty", "cutlass"))
    env = os.environ.get("CUTLASS_PATH")
    if env:
        roots.insert(0, env)
    for r in roots:
        if os.path.exists(os.path.join(r, "include", "cutlass", "cutlass.h")) and \
                os.path.exists(os.path.join(r, "tools", "util", "include", "cutlass", "util", "reference", "host", "gemm.h")):
            return r
    return None


def build(force: bool = False):
    """Returns the binary's path, or None (with a reason printed) when CUTLASS or nvcc is not available."""
    if not force and os.path.exists(BINARY) and os.path.getmtime(BINARY) >= os.path.getmtime(SOURCE):
        return BINARY
    root = find_cutlass()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if root is None or not os.path.exists(nvcc):
        print("oracle/_ref not built:", "no CUTLASS copy with host reference utilities found" if root is None else "nvcc not found")
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [nvcc, "-O2", "-std=c++17", "-w", f"-I{root}/include", f"-I{root}/tools/util/include", "-x", "cu", SOURCE, "-o", BINARY]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        print("oracle/_ref not built: compile failed\n" + r.stderr[-2000:])
        return None
    return BINARY


def run(m: int, n: int, k: int, seed: int = 3080):
    """(seconds, GFLOP/s, checksum) of one host GEMM, or None if the binary is not there."""
    if not os.path.exists(BINARY):
        return None
    out = subprocess.run([BINARY, str(m), str(n), str(k), str(seed)], capture_output=True, text=True, timeout=600).stdout.split()
    return float(out[0]), float(out[1]), float(out[2])


def inputs(m: int, n: int, k: int, seed: int = 3080):
    """The harness's operands, regenerated bit for bit: dense A (m, k) of {-1, 0, +1} with a 2:4 pattern and
    B (k, n) of integers in [-8, 8], both float16."""
    import numpy as np
    mask = (1 << 64) - 1
    state = seed

    def nxt():
        nonlocal state
        state = (state + 0x9E3779B97F4A7C15) & mask
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)

    pairs = [(0, 1), (0, 2), (1, 2), (0, 3), (1, 3), (2, 3)]
    A = np.zeros((m, k), np.float16)
    for i in range(m):
        for g in range(k // 4):
            r = nxt()
            p = pairs[r % 6]
            A[i, 4 * g + p[0]] = 1.0 if (r >> 8) & 1 else -1.0
            A[i, 4 * g + p[1]] = 1.0 if (r >> 9) & 1 else -1.0
    B = np.array([float(int(nxt() % 17) - 8) for _ in range(k * n)], np.float16).reshape(k, n)
    return A, B


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
