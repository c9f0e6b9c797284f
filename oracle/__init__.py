"""CPU oracle: TEST INFRASTRUCTURE, not product code.

numpy-facing wrapper around ``oracle/onebit_oracle.c`` (a plain-C restatement of the reference's
algorithm for ``C = A_sparse x B``). Only ``tests/``, the smoke check and the benchmark's CPU
baseline legs import this package; the shipped library never does.

Parity status: pinned. ``tests/test_oracle.py`` checks these functions against golden vectors made
by executing the reference's Python (``tests/golden/make_golden.py``) and against the known-answer
rows of the reference's ``tests/python/test_sparse.py:48-68``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_HERE, "_build")
_SO = os.path.join(_BUILD, "libonebit_oracle.so")
_SRC = os.path.join(_HERE, "onebit_oracle.c")

META_PYTHON, META_CUTLASS = 0, 1
DENSE_F16, DENSE_BF16, DENSE_I32 = 0, 1, 2

_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with gcc (OpenMP on) into oracle/_build/."""
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(_SRC):
        return _SO
    os.makedirs(_BUILD, exist_ok=True)
    subprocess.check_call(
        ["gcc", "-O3", "-march=x86-64-v2", "-fopenmp", "-shared", "-fPIC", "-o", _SO, _SRC])
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def max_threads() -> int:
    return int(lib().ob_oracle_max_threads())


def _dense_dtype(dense: np.ndarray, dtype_code: int | None) -> int:
    if dtype_code is not None:
        return dtype_code
    if dense.dtype == np.float16:
        return DENSE_F16
    if dense.dtype == np.int32:
        return DENSE_I32
    raise TypeError("pass bf16 as its uint16 bit pattern with dtype_code=DENSE_BF16")


def compress(dense: np.ndarray, dtype_code: int | None = None):
    """dense (m,k) -> (canonical meta uint16 (m,k/16), signs uint8 (m,k/2), kept values (m,k/2))."""
    code = _dense_dtype(dense, dtype_code)
    dense = np.ascontiguousarray(dense)
    m, k = dense.shape
    meta = np.zeros((m, k // 16), np.uint16)
    signs = np.zeros((m, k // 2), np.uint8)
    sparse = np.zeros((m, k // 2), dense.dtype)
    lib().ob_oracle_compress(_p(dense), code, ctypes.c_int64(m), ctypes.c_int64(k), _p(meta), _p(signs), _p(sparse))
    return meta, signs, sparse


def meta_reorder(canon: np.ndarray, dialect: int) -> np.ndarray:
    canon = np.ascontiguousarray(canon, np.uint16)
    m, nc = canon.shape
    if m % (64 if dialect == META_PYTHON else 32) != 0:
        raise ValueError(f"{m} rows: the metadata shuffle works on whole groups of {64 if dialect == META_PYTHON else 32} rows")
    out = np.zeros((m, nc), np.uint16)
    lib().ob_oracle_meta_reorder(_p(canon), dialect, ctypes.c_int64(m), ctypes.c_int64(nc), _p(out))
    return out


def meta_unreorder(meta: np.ndarray, dialect: int) -> np.ndarray:
    meta = np.ascontiguousarray(meta).view(np.uint16)
    m, nc = meta.shape
    if m % (64 if dialect == META_PYTHON else 32) != 0:
        raise ValueError(f"{m} rows: the metadata shuffle works on whole groups of {64 if dialect == META_PYTHON else 32} rows")
    out = np.zeros((m, nc), np.uint16)
    lib().ob_oracle_meta_unreorder(_p(meta), dialect, ctypes.c_int64(m), ctypes.c_int64(nc), _p(out))
    return out


def pack_bits(signs: np.ndarray) -> np.ndarray:
    """signs (m, k/2) of 0/1 -> reference A bitfield uint8 (k/2, m/8)."""
    signs = np.ascontiguousarray(signs, np.uint8)
    m, kh = signs.shape
    out = np.zeros((kh, m // 8), np.uint8)
    lib().ob_oracle_pack_bits(_p(signs), ctypes.c_int64(m), ctypes.c_int64(kh), _p(out))
    return out


def unpack_bits(bitfield: np.ndarray, m: int) -> np.ndarray:
    bitfield = np.ascontiguousarray(bitfield, np.uint8)
    kh = bitfield.size // (m // 8)
    out = np.zeros((m, kh), np.uint8)
    lib().ob_oracle_unpack_bits(_p(bitfield), ctypes.c_int64(m), ctypes.c_int64(kh), _p(out))
    return out


def pack(dense: np.ndarray, dialect: int = META_PYTHON, dtype_code: int | None = None):
    """The whole reference pack step after masking: dense -> (A bitfield, reference-ordered meta int16)."""
    canon, signs, _ = compress(dense, dtype_code)
    return pack_bits(signs), meta_reorder(canon, dialect).view(np.int16)


def dequant(bitfield: np.ndarray, meta: np.ndarray, dialect: int, m: int, k: int) -> np.ndarray:
    bitfield = np.ascontiguousarray(bitfield, np.uint8)
    meta = np.ascontiguousarray(meta).view(np.uint16)
    out = np.zeros((m, k), np.int8)
    lib().ob_oracle_dequant(_p(bitfield), _p(meta), dialect, ctypes.c_int64(m), ctypes.c_int64(k), _p(out))
    return out


def gemm(bitfield: np.ndarray, meta: np.ndarray, dialect: int, B: np.ndarray, m: int,
         scale: np.ndarray | None = None, threads: int = 0):
    """Returns (C fp32 (m,n), C fp16 (m,n)) for B fp16 (k,n)."""
    bitfield = np.ascontiguousarray(bitfield, np.uint8)
    meta = np.ascontiguousarray(meta).view(np.uint16)
    B = np.ascontiguousarray(B, np.float16)
    k, n = B.shape
    if scale is not None:
        scale = np.ascontiguousarray(scale, np.float16)
    o32 = np.zeros((m, n), np.float32)
    o16 = np.zeros((m, n), np.float16)
    lib().ob_oracle_gemm(_p(bitfield), _p(meta), dialect, _p(scale), _p(B), ctypes.c_int64(m),
                         ctypes.c_int64(n), ctypes.c_int64(k), _p(o32), _p(o16), int(threads))
    return o32, o16


def mask24(dense: np.ndarray) -> np.ndarray:
    dense = np.ascontiguousarray(dense, np.float16)
    m, k = dense.shape
    out = np.zeros((m, k), np.uint8)
    lib().ob_oracle_mask24(_p(dense), ctypes.c_int64(m), ctypes.c_int64(k), _p(out))
    return out
