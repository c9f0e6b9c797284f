"""Pipeline timelines of the GEMM kernels, for tuning.

    python -m onebitsparsemul_b200.trace prefill  <a_rows> <n> <a_cols>     # CTA-pair / single-CTA tcgen05 kernel
    python -m onebitsparsemul_b200.trace decode   <a_rows> <n> <a_cols>     # split-K cluster kernel

Builds a second copy of the library with -DOB_TRACE (onebitsparsemul_b200/build/libonebitmul_trace.so),
in which one CTA (pair) in the middle of the grid records the SM clock at every hand-over of its
pipeline, runs the GEMM a few times and prints the recorded cycle counts relative to the kernel's
start. The production library contains none of this. ONEBIT_PREFILL_VARIANT selects the tcgen05
kernel variant as usual.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import sys

import numpy as np

from . import _lib, build

TRACE_LIB = os.path.join(build.HERE, "build", "libonebitmul_trace.so")


def build_trace_library() -> str:
    srcs = [os.path.join(build.CSRC, f) for f in build.SOURCES]
    deps = srcs + [os.path.join(build.CSRC, f) for f in os.listdir(build.CSRC) if f.endswith(".h")]
    if os.path.exists(TRACE_LIB) and all(os.path.getmtime(d) <= os.path.getmtime(TRACE_LIB) for d in deps):
        return TRACE_LIB
    os.makedirs(os.path.dirname(TRACE_LIB), exist_ok=True)
    subprocess.check_call([build.nvcc(), *build.NVCC_FLAGS, "-DOB_TRACE", "-shared", "-o", TRACE_LIB, *srcs, "-lcudart"])
    return TRACE_LIB


def _packed_problem(m, k):
    import torch

    import onebitsparsemul_b200 as ob
    w = torch.zeros((m, k // 4, 4), dtype=torch.float16, device="cuda")
    w[..., 0], w[..., 2] = 1.0, -1.0
    return ob.pack_weight(w.reshape(m, k), apply_mask=False, keep_reference=False)


def trace_prefill(m, n, k):
    import torch

    import onebitsparsemul_b200 as ob
    lib = _lib.load()
    pw = _packed_problem(m, k)
    B = torch.randn((k, n), device="cuda", dtype=torch.float16)
    C = torch.empty((m, n), dtype=torch.float16, device="cuda")
    for _ in range(3):
        ob.matmul_packed(pw, B, out=C, kernel=_lib.KERNEL_PREFILL)
    torch.cuda.synchronize()
    kt = k // 128
    pair = np.zeros((16, 512), np.int64)
    single = np.zeros((8, 512), np.int64)
    for name, buf in (("onebit_debug_read_trace2", pair), ("onebit_debug_read_trace", single)):
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = [ctypes.c_void_p], ctypes.c_int
        fn(buf.ctypes.data)
    pers = np.zeros((16, 512), np.int64)
    fn = lib.onebit_debug_read_trace3
    fn.argtypes, fn.restype = [ctypes.c_void_p], ctypes.c_int
    fn(pers.ctypes.data)
    if pers[7, 0] != 0:                                    # the persistent CTA-pair kernel ran
        for c in (0, 1):
            b = pers[8 * c:8 * c + 8]
            t0 = b[7, 0]
            print(f"CTA {c} of the traced cluster: kernel end {b[7, 1] - t0}")
            print("  tile  MMA:accumulator free  MMA:tile committed  epilogue:accumulator full  epilogue:drained  epilogue:stored")
            for tl in range(16):
                if b[2, tl] == 0:
                    break
                print(f"  {tl:4d} " + "  ".join(f"{(b[e, tl] - t0) if b[e, tl] else 0:20d}" for e in (0, 1, 2, 3, 4)))
        return
    if pair[7, 2] != 0:                                    # the CTA-pair kernel ran
        for c in (0, 1):
            b = pair[8 * c:8 * c + 8]
            t0 = b[7, 2]
            print(f"CTA {c} of the traced pair: barriers ready {b[7, 4] - t0}, accumulator ready {b[7, 0] - t0}, "
                  f"epilogue {b[7, 1] - b[7, 0]} cycles")
            print("  it  producer:stage free  expander:stage landed  expander:arrived  MMA:operands ready  MMA:issued")
            its = [i for i in list(range(0, 8)) + list(range(max(8, kt // 2 - 4), kt // 2)) if b[1, i] != 0]
            for it in its:
                print(f"  {it:3d} " + "  ".join(f"{(b[e, it] - t0) if b[e, it] else 0:18d}" for e in (0, 1, 3, 5, 6)))
        d = np.diff(pair[6, :kt][pair[6, :kt] != 0])
        if len(d) > 4:
            print("leader MMA thread, cycles per pipeline iteration: median", float(np.median(d[2:])))
    else:
        b, t0 = single, single[7, 2]
        print(f"accumulator ready {b[7, 0] - t0}, epilogue {b[7, 1] - b[7, 0]}, whole CTA {b[7, 3] - t0} cycles")
        print("  it  producer:stage free  expander:stage landed  expander:slot free  expander:arrived  MMA:operands ready  MMA:issued")
        for it in list(range(0, 8)) + list(range(max(8, kt - 4), kt)):
            print(f"  {it:3d} " + "  ".join(f"{b[e, it] - t0:18d}" for e in (0, 1, 2, 3, 5, 6)))
        d = np.diff(b[6, :kt])
        print("MMA thread, cycles per pipeline iteration: median", float(np.median(d[4:])))


def trace_decode(m, n, k):
    import torch

    import onebitsparsemul_b200 as ob
    lib = _lib.load()
    pw = _packed_problem(m, k)
    B = torch.randn((k, n), device="cuda", dtype=torch.float16)
    C = torch.empty((m, n), dtype=torch.float16, device="cuda")
    for _ in range(5):
        ob.matmul_packed(pw, B, out=C, kernel=_lib.KERNEL_DECODE)
    torch.cuda.synchronize()
    buf = np.zeros((4, 16), np.int64)
    fn = lib.onebit_debug_read_trace_decode
    fn.argtypes, fn.restype = [ctypes.c_void_p], ctypes.c_int
    fn(buf.ctypes.data)
    names = ["start", "weight loads issued", "tokens staged", "half barrier", "MMAs done", "partials pushed", "cluster barrier", "stored"]
    for i, who in enumerate(["CTA 0 thread 0", "CTA 0 thread 511", "CTA 1 thread 0", "CTA 1 thread 511"]):
        print(who + ": " + ", ".join(f"{names[e]} {buf[i, e] - buf[i, 0]}" for e in range(1, 8)))
        chunks = [f"chunk {c}: weights landed {buf[i, 8 + 2 * c] - buf[i, 0]}, multiplied {buf[i, 9 + 2 * c] - buf[i, 0]}"
                  for c in range(4) if buf[i, 8 + 2 * c]]
        if chunks:
            print("    " + "; ".join(chunks))


def main(argv):
    if len(argv) != 5 or argv[1] not in ("prefill", "decode"):
        print(__doc__)
        return 2
    _lib.LIB_PATH = build_trace_library()
    m, n, k = int(argv[2]), int(argv[3]), int(argv[4])
    (trace_prefill if argv[1] == "prefill" else trace_decode)(m, n, k)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
