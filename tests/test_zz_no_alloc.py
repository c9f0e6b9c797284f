"""The allocation-free entry point, onebit_sparse_matmul_static.

Some hosts of this library cannot call cudaMalloc once they are running: a serving process whose own
memory pool has claimed the whole GPU, or a token-by-token decode loop that cannot absorb the
device-wide stall an allocation causes. For them the library carries its relayout scratch inside
its own image. This file checks, through the C ABI, that the entry point gives the same answer as the
ordinary stateless entry point (onebit_sparse_matmul_ex), twice in a row with different weights so
that nothing left in the shared array by the first call can leak into the second; that it also
agrees with the CPU oracle (exactly, on integer tokens); that the free device memory reported by the
driver does not move across a call once the per-device warm-up call has been made; and that it
refuses problems larger than its fixed array. It is named to be collected last: a run that stops at
the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

import oracle
from onebitsparsemul_b200 import _lib
from tests import helpers

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def operands(seed, m, k, n, dialect):
    rng = np.random.default_rng(seed)
    dense, scale = helpers.make_weights(rng, m, k)
    canon, signs, _ = oracle.compress(dense)
    B = helpers.make_tokens(rng, k, n)
    return (dev(oracle.pack_bits(signs)), dev(oracle.meta_reorder(canon, dialect).view(np.int16)), dev(scale), dev(B))


def test_static_entry_point_matches_the_allocating_one_twice_in_a_row():
    assert torch.cuda.is_available()
    lib = _lib.load()
    # two different problems back to back: the second is smaller, so stale bytes of the first stay
    # in the array behind it, and uses the other metadata order and more tokens
    for seed, (m, k, n, dialect, out_code, out_dtype) in enumerate([
            (512, 1024, 4, _lib.META_PYTHON, _lib.OUT_F16, torch.float16),
            (256, 384, 24, _lib.META_CUTLASS, _lib.OUT_F32, torch.float32)]):
        a_bits, e_meta, scale, B = operands(900 + seed, m, k, n, dialect)
        want = torch.zeros((m, n), dtype=out_dtype, device="cuda")
        ws = torch.zeros(lib.onebit_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")
        _lib.check(lib.onebit_sparse_matmul_ex(a_bits.data_ptr(), B.data_ptr(), want.data_ptr(), e_meta.data_ptr(),
                                               scale.data_ptr(), m, n, k, out_code, dialect, ws.data_ptr(), ws.numel(), None))
        got = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
        _lib.check(lib.onebit_sparse_matmul_static(a_bits.data_ptr(), B.data_ptr(), got.data_ptr(), e_meta.data_ptr(),
                                                   scale.data_ptr(), m, n, k, out_code, dialect, None))
        torch.cuda.synchronize()
        _lib.check(lib.onebit_check_device_status())
        got_np, want_np = got.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(got_np).all()
        # same bound as the GEMM parity tests: max |err| <= 1e-2 * |row|_inf (n = 24 takes the
        # tensor-memory kernel in the allocating entry point and the cluster kernel here)
        ok, worst = helpers.row_tolerance_ok(got_np, want_np.astype(np.float32))
        assert ok, f"worst err / bound = {worst}"
        if n <= 16:
            assert (got_np == want_np).all()          # same kernel on both sides: identical bits


def test_static_entry_point_is_exact_against_the_oracle_and_allocates_nothing():
    assert torch.cuda.is_available()
    lib = _lib.load()
    m, k, n, dialect = 384, 640, 8, _lib.META_PYTHON
    rng = np.random.default_rng(77)
    dense, _ = helpers.make_weights(rng, m, k)
    canon, signs, _ = oracle.compress(dense)
    bits, meta = oracle.pack_bits(signs), oracle.meta_reorder(canon, dialect)
    B = helpers.make_tokens(rng, k, n, "int")            # integer tokens: every partial sum is exact in fp32
    want, _ = oracle.gemm(bits, meta, dialect, B, m, scale=None)
    a_bits, e_meta, Bd = dev(bits), dev(meta.view(np.int16)), dev(B)
    got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")

    def call():
        _lib.check(lib.onebit_sparse_matmul_static(a_bits.data_ptr(), Bd.data_ptr(), got.data_ptr(), e_meta.data_ptr(),
                                                   None, m, n, k, _lib.OUT_F32, dialect, None))
        torch.cuda.synchronize()

    call()                                               # the per-device warm-up: address look-up, module load
    assert (got.cpu().numpy() == want).all()
    free_before, _ = torch.cuda.mem_get_info()
    got.fill_(float("nan"))                              # in place: no allocation of the test's own in between
    call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory moved by {free_before - free_after} bytes across the call"
    assert (got.cpu().numpy() == want).all()
    _lib.check(lib.onebit_check_device_status())


def test_static_entry_point_rejects_oversize_and_bad_shapes():
    lib = _lib.load()
    p = 256                                            # never dereferenced: validation fails first
    assert lib.onebit_sparse_matmul_static(p, p, p, p, None, 8192, 8, 8192, 0, 0, None) == 4
    assert b"exceeds the built-in scratch" in lib.onebit_last_error()
    # sizes whose product wraps around 64 bits are refused as well
    assert lib.onebit_sparse_matmul_static(p, p, p, p, None, 1 << 33, 8, 1 << 31, 0, 0, None) == 4
    assert lib.onebit_sparse_matmul_static(p, p, p, p, None, 100, 8, 128, 0, 0, None) == 1
    assert lib.onebit_sparse_matmul_static(None, p, p, p, None, 128, 8, 128, 0, 0, None) == 2
