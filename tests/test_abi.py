"""The C-ABI library: loads, exports every declared symbol, rejects bad calls on the host (CPU only;
no compute call is made)."""
import ctypes
import os
import re
import subprocess

import pytest

from onebitsparsemul_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build_library()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "onebit_sparse_tensor.h")).read()
    body = text[text.index('extern "C" {'):]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    return sorted(set(re.findall(r"\b(onebit_\w+)\s*\(", body)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert "onebit_sparse_matmul_ex" in names and "onebit_pack_from_dense" in names and len(names) >= 10
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures and header disagree"
    for name in names:
        assert getattr(lib, name) is not None


def test_reference_symbol_keeps_its_mangled_name(lib):
    # the reference declares onebit_sparse_matmul with C++ linkage (include/onebit_sparse_tensor.h:5)
    out = subprocess.check_output(["nm", "-D", "--defined-only", _lib.LIB_PATH], text=True)
    assert " T _Z20onebit_sparse_matmulPvS_S_S_S_iii" in out
    assert getattr(lib, _lib.LEGACY_SYMBOL) is not None


def test_size_queries(lib):
    assert lib.onebit_packed_bits_bytes(4096, 4096) == 4096 * 4096 // 16
    assert lib.onebit_packed_meta_bytes(4096, 4096) == 4096 * 4096 // 8
    assert lib.onebit_workspace_bytes(128, 128) == 1024 + 2048


def test_host_side_validation_needs_no_gpu(lib):
    p = ctypes.c_void_p(256)          # never dereferenced: validation fails first
    assert lib.onebit_relayout(None, p, 0, 128, 128, p, p, None) == 2
    assert b"null" in lib.onebit_last_error()
    assert lib.onebit_relayout(p, p, 0, 100, 128, p, p, None) == 1
    assert lib.onebit_matmul_packed(p, p, None, p, p, 128, 0, 128, 0, 0, None) == 1
    assert lib.onebit_matmul_packed(p, p, None, p, p, 128, 8, 128, 7, 0, None) == 5
    assert lib.onebit_sparse_matmul_ex(p, p, p, p, None, 96, 8, 64, 0, _lib.META_PYTHON, None, 0, None) == 1
    assert b"multiple of 64" in lib.onebit_last_error()
    assert lib.onebit_sparse_matmul_ex(p, p, p, p, None, 128, 8, 128, 0, 1, p, 16, None) == 4
    assert lib.onebit_pack_from_dense(p, 9, 128, 128, None, None, None, 0, None, None, None) == 5
    assert lib.onebit_pack_from_dense(p, 0, 64, 64, None, None, None, 0, p, p, None) == 1
    assert lib.onebit_mask24(p, 12, None, None, None) == 1


def test_python_layer_refuses_to_run_without_cuda():
    import torch

    import onebitsparsemul_b200 as ob
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(ob.OneBitError):
        ob.cuda_binary_mul(torch.zeros((64, 16), dtype=torch.uint8), torch.zeros((128, 8), dtype=torch.float16),
                           torch.zeros((128, 8), dtype=torch.int16))
