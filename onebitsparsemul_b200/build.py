"""Build recipe of libonebitmul.so: explicit nvcc for sm_100a, in-tree output.

The shared library lands next to this file (onebitsparsemul_b200/libonebitmul.so) so that it
travels with the source tree; nothing is installed into site-packages or a JIT cache.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libonebitmul.so")
SOURCES = ["api.cu", "pack.cu", "mask.cu", "relayout.cu", "gemm_simple.cu", "gemm_decode.cu", "gemm_decode_sm100.cu", "gemm_prefill_sm100.cu", "gemm_prefill2_sm100.cu", "gemm_prefill3_sm100.cu", "gemm_prefill_splitk_sm100.cu", "noalloc.cu", "host_pipeline.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libonebitmul.so cannot be built")
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu of csrc/ to an object and link libonebitmul.so. Returns its path."""
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".h")]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "onebit_sparse_tensor.h"))
    objs, procs = [], []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [nvcc(), *NVCC_FLAGS, "-c", s, "-o", o] + (["-Xptxas", "-v"] if verbose else [])
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            print(f"--- {src}\n{out}")
        if p.returncode != 0:
            failed.append(src)
    if failed:
        raise RuntimeError(f"nvcc failed for {failed}")
    if force or procs or _stale(LIB, objs):
        subprocess.check_call([nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"])
    return LIB


def build_torch_extension(force: bool = False) -> str:
    """Compile the `onebit_sparse_cuda` torch extension (host C++ only) next to the package and
    link it against libonebitmul.so. Returns the module path."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    lib = build_library()
    root = os.path.dirname(HERE)
    src = os.path.join(CSRC, "torch_kernel_cuda.cpp")
    out = os.path.join(root, "onebit_sparse_cuda" + sysconfig.get_config_var("EXT_SUFFIX"))
    hdr = os.path.join(root, "include", "onebit_sparse_tensor.h")
    if not force and not _stale(out, [src, hdr, lib]):
        return out
    inc = [f"-I{p}" for p in cpp_extension.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}",
                                                                  f"-I{os.path.join(root, 'include')}"]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=onebit_sparse_cuda",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *inc, src, "-o", out, f"-L{HERE}", "-lonebitmul", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_python",
           "-lc10", "-lc10_cuda", "-ltorch_cuda", f"-Wl,-rpath,$ORIGIN/{os.path.basename(HERE)}", f"-Wl,-rpath,{torch_lib}"]
    subprocess.check_call(cmd)
    return out


def build_cli(force: bool = False) -> str:
    """Compile the benchmark CLI (the reference's `a.out`) at the repository root."""
    lib = build_library()
    root = os.path.dirname(HERE)
    src = os.path.join(CSRC, "kernel_test.cu")
    out = os.path.join(root, "a.out")
    if not os.path.exists(src):
        return ""
    if not force and not _stale(out, [src, lib, os.path.join(root, "include", "onebit_sparse_tensor.h")]):
        return out
    subprocess.check_call([nvcc(), *NVCC_FLAGS, f"-I{os.path.join(root, 'include')}", src, "-o", out, f"-L{HERE}",
                           "-lonebitmul", "-Xlinker", f"-rpath=$ORIGIN/{os.path.basename(HERE)}"])
    return out


if __name__ == "__main__":
    import sys
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--all" in sys.argv:
        print(build_torch_extension(force="--force" in sys.argv))
        print(build_cli(force="--force" in sys.argv))
