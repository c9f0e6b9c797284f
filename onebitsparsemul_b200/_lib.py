"""ctypes binding of libonebitmul.so (the C ABI declared in include/onebit_sparse_tensor.h).

There is no CPU implementation behind this module: if the shared library has not been built, or it
cannot be loaded, importing the symbols fails loudly.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libonebitmul.so")

META_PYTHON, META_CUTLASS = 0, 1
OUT_F32, OUT_F16 = 0, 1
DENSE_F16, DENSE_BF16, DENSE_I32 = 0, 1, 2
KERNEL_AUTO, KERNEL_PREFILL, KERNEL_DECODE = 0, 1, 2
KERNEL_STABLE_WEIGHTS = 0x100     # flag OR-ed into a kernel selector (see the header)

# every extern "C" symbol of include/onebit_sparse_tensor.h, with its ctypes signature
_vp, _i64, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
SIGNATURES = {
    "onebit_last_error": (ctypes.c_char_p, []),
    "onebit_packed_bits_bytes": (_sz, [_i64, _i64]),
    "onebit_packed_meta_bytes": (_sz, [_i64, _i64]),
    "onebit_workspace_bytes": (_sz, [_i64, _i64]),
    "onebit_sparse_matmul_ex": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp, _sz, _vp]),
    "onebit_sparse_matmul_static": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "onebit_relayout": (_int, [_vp, _vp, _int, _i64, _i64, _vp, _vp, _vp]),
    "onebit_matmul_packed": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "onebit_linear_tokens": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "onebit_host_workspace_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "onebit_copy_2d_async": (_int, [_vp, _sz, _vp, _sz, _sz, _sz, _vp]),
    "onebit_matmul_packed_scatter": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _int, _i64, _i64, _i64, _vp]),
    "onebit_matmul_packed_host": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "onebit_pack_from_dense": (_int, [_vp, _int, _i64, _i64, _vp, _vp, _vp, _int, _vp, _vp, _vp]),
    "onebit_mask_pack_from_dense": (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _int, _vp, _vp, _vp]),
    "onebit_mask24": (_int, [_vp, _i64, _vp, _vp, _vp]),
    "onebit_unpack_to_dense": (_int, [_vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "onebit_check_device_status": (_int, []),
}
# the reference's own entry point keeps its C++-mangled name
LEGACY_SYMBOL = "_Z20onebit_sparse_matmulPvS_S_S_S_iii"

_lib = None


class OneBitError(RuntimeError):
    """A call into libonebitmul failed; the message is onebit_last_error()."""


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m onebitsparsemul_b200.build` (or `make share_lib`). "
            "There is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    legacy = getattr(lib, LEGACY_SYMBOL)
    legacy.restype = None
    legacy.argtypes = [_vp, _vp, _vp, _vp, _vp, _int, _int, _int]
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != 0:
        raise OneBitError(f"libonebitmul error {rc}: {load().onebit_last_error().decode()}")
