"""GEMM parity through the C ABI: every kernel against the CPU oracle on the same seeded inputs.

Integer-valued tokens (the reference CLI's fixture, tests/kernel_test.cu:321-332) make every partial
sum exact, so those cases are compared bit for bit; normally distributed tokens are held to the
path's stated bound, max |err| <= 1e-2 * |row|_inf on the fp16 output with fp32 accumulation.
"""
import numpy as np
import pytest
import torch

import oracle
from onebitsparsemul_b200 import _lib
from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    assert torch.cuda.is_available()
    return _lib.load()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


class Problem:
    """Seeded weights in every order the ABI takes, on host and device."""

    def __init__(self, seed, m, k, dialect=_lib.META_PYTHON):
        rng = np.random.default_rng(seed)
        self.m, self.k, self.dialect, self.rng = m, k, dialect, rng
        self.dense, self.scale = helpers.make_weights(rng, m, k)
        canon, signs, _ = oracle.compress(self.dense)
        self.a_bits, self.e_meta = oracle.pack_bits(signs), oracle.meta_reorder(canon, dialect)
        self.d_bits, self.d_meta, self.d_scale = dev(self.a_bits), dev(self.e_meta.view(np.int16)), dev(self.scale)
        if m % 128 == 0 and k % 128 == 0:
            bt, mt = helpers.tile_order_from_canonical(canon, signs)
            self.d_bits_tile, self.d_meta_tile = dev(bt), dev(mt)

    def oracle(self, B, use_scale):
        return oracle.gemm(self.a_bits, self.e_meta, self.dialect, B, self.m, scale=self.scale if use_scale else None)


def run_packed(lib, p, B, out_dtype, kernel, use_scale):
    d_b = dev(B)
    out = torch.full((p.m, B.shape[1]), float("nan"), dtype=out_dtype, device="cuda")
    _lib.check(lib.onebit_matmul_packed(p.d_bits_tile.data_ptr(), p.d_meta_tile.data_ptr(),
                                        p.d_scale.data_ptr() if use_scale else None, d_b.data_ptr(), out.data_ptr(),
                                        p.m, B.shape[1], p.k, _lib.OUT_F16 if out_dtype == torch.float16 else _lib.OUT_F32,
                                        kernel, None))
    _lib.check(lib.onebit_check_device_status())
    return out.cpu().numpy()


def check_exact_and_tolerance(lib, p, n, kernel, sigma=1.0):
    # exact: integer tokens, no scale, fp32 out
    B = helpers.make_tokens(p.rng, p.k, n, "int")
    want32, _ = p.oracle(B, use_scale=False)
    got = run_packed(lib, p, B, torch.float32, kernel, use_scale=False)
    assert (got == want32).all(), f"max abs diff {np.abs(got - want32).max()}"
    # tolerance: normal tokens, per-row scale, fp16 out
    B = helpers.make_tokens(p.rng, p.k, n, "normal", sigma)
    want32, want16 = p.oracle(B, use_scale=True)
    got = run_packed(lib, p, B, torch.float16, kernel, use_scale=True)
    ok, worst = helpers.row_tolerance_ok(got, want32)
    assert ok, f"worst err / bound = {worst}"
    assert np.isfinite(got).all()


# ---- plain kernel on the reference orders: bit-exact in every case (same summation order) ------------

@pytest.mark.parametrize("m,n,k,dialect", [(64, 8, 64, _lib.META_PYTHON), (192, 5, 96, _lib.META_PYTHON),
                                           (96, 33, 160, _lib.META_CUTLASS), (32, 1, 32, _lib.META_CUTLASS)])
def test_plain_kernel_bit_exact(lib, m, n, k, dialect):
    p = Problem(11 + m, m, k, dialect)
    B = helpers.make_tokens(p.rng, k, n)
    want32, want16 = p.oracle(B, use_scale=True)
    d_b = dev(B)
    for dtype, want, code in ((torch.float32, want32, _lib.OUT_F32), (torch.float16, want16, _lib.OUT_F16)):
        out = torch.zeros((m, n), dtype=dtype, device="cuda")
        _lib.check(lib.onebit_sparse_matmul_ex(p.d_bits.data_ptr(), d_b.data_ptr(), out.data_ptr(), p.d_meta.data_ptr(),
                                               p.d_scale.data_ptr(), m, n, k, code, dialect, None, 0, None))
        assert (out.cpu().numpy() == want).all()


# ---- decode kernel: config 2 shapes (7B-class linear layers), n in {1, 4, 8, 16} ------------------------

@pytest.mark.parametrize("m,k", [(4096, 4096), (11008, 4096), (4096, 11008)])
@pytest.mark.parametrize("n", [1, 4, 8, 16])
def test_decode_kernel_config2(lib, m, k, n):
    check_exact_and_tolerance(lib, Problem(m + k + n, m, k), n, _lib.KERNEL_DECODE)


@pytest.mark.parametrize("m,n,k", [(128, 1, 128), (128, 3, 256), (256, 16, 1152), (384, 40, 640), (128, 9, 128 * 37)])
def test_decode_kernel_ragged(lib, m, n, k):
    check_exact_and_tolerance(lib, Problem(m * 3 + k + n, m, k), n, _lib.KERNEL_DECODE)


# ---- tensor-memory kernel: config 0, reduced config 1 / 3 shapes, ragged n -------------------------------

@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (128, 128, 512), (512, 512, 512), (1024, 1024, 1024),
                                   (256, 2048, 1024), (2048, 2048, 2048)])
def test_prefill_kernel_squares(lib, m, n, k):
    check_exact_and_tolerance(lib, Problem(m + n + k, m, k), n, _lib.KERNEL_PREFILL, sigma=0.5 if n == 2048 else 1.0)


@pytest.mark.parametrize("m,n,k", [(128, 8, 128), (128, 24, 256), (256, 72, 384), (128, 200, 640), (384, 136, 128)])
def test_prefill_kernel_ragged_n(lib, m, n, k):
    check_exact_and_tolerance(lib, Problem(m + 5 * n + k, m, k), n, _lib.KERNEL_PREFILL)


# ---- dispatcher and the stateless entry points ---------------------------------------------------------------

@pytest.mark.parametrize("n", [1, 16, 17, 64])
@pytest.mark.parametrize("dialect", [_lib.META_PYTHON, _lib.META_CUTLASS])
def test_stateless_entry_point_dispatch(lib, n, dialect):
    m, k = 256, 512
    p = Problem(100 + n, m, k, dialect)
    B = helpers.make_tokens(p.rng, k, n, "int")
    want32, _ = p.oracle(B, use_scale=False)
    d_b = dev(B)
    out = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    ws = torch.zeros(lib.onebit_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")
    _lib.check(lib.onebit_sparse_matmul_ex(p.d_bits.data_ptr(), d_b.data_ptr(), out.data_ptr(), p.d_meta.data_ptr(), None,
                                           m, n, k, _lib.OUT_F32, dialect, ws.data_ptr(), ws.numel(), None))
    _lib.check(lib.onebit_check_device_status())
    assert (out.cpu().numpy() == want32).all()
    # library-owned scratch
    out.zero_()
    _lib.check(lib.onebit_sparse_matmul_ex(p.d_bits.data_ptr(), d_b.data_ptr(), out.data_ptr(), p.d_meta.data_ptr(), None,
                                           m, n, k, _lib.OUT_F32, dialect, None, 0, None))
    _lib.check(lib.onebit_check_device_status())
    assert (out.cpu().numpy() == want32).all()


def test_two_streams_share_the_library_scratch(lib):
    # workspace == NULL on two non-blocking streams with different weights: the library orders the two calls'
    # use of its one scratch block on the GPU, so both results are exact
    m, n, k = 1024, 64, 2048
    probs = [Problem(500 + i, m, k) for i in range(2)]
    Bs = [helpers.make_tokens(p.rng, k, n, "int") for p in probs]
    wants = [p.oracle(B, use_scale=False)[0] for p, B in zip(probs, Bs)]
    d_bs = [dev(B) for B in Bs]
    outs = [torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda") for _ in probs]
    streams = [torch.cuda.Stream() for _ in probs]
    torch.cuda.synchronize()
    for rep in range(3):
        for p, d_b, out, st in zip(probs, d_bs, outs, streams):
            _lib.check(lib.onebit_sparse_matmul_ex(p.d_bits.data_ptr(), d_b.data_ptr(), out.data_ptr(), p.d_meta.data_ptr(), None,
                                                   m, n, k, _lib.OUT_F32, p.dialect, None, 0, st.cuda_stream))
    torch.cuda.synchronize()
    _lib.check(lib.onebit_check_device_status())
    for out, want in zip(outs, wants):
        assert (out.cpu().numpy() == want).all()


def test_single_token_from_an_unaligned_address(lib):
    # B (k, 1) that starts 2 bytes into a buffer is legal fp16: the kernel must not use 16-byte loads on it
    m, k = 256, 512
    p = Problem(41, m, k)
    B = helpers.make_tokens(p.rng, k, 1, "int")
    want32, _ = p.oracle(B, use_scale=False)
    buf = torch.zeros(k + 8, dtype=torch.float16, device="cuda")
    buf[1:k + 1] = dev(B).reshape(-1)
    out = torch.full((m, 1), float("nan"), dtype=torch.float32, device="cuda")
    _lib.check(lib.onebit_matmul_packed(p.d_bits_tile.data_ptr(), p.d_meta_tile.data_ptr(), None, buf.data_ptr() + 2,
                                        out.data_ptr(), m, 1, k, _lib.OUT_F32, _lib.KERNEL_DECODE, None))
    _lib.check(lib.onebit_check_device_status())
    assert (out.cpu().numpy() == want32).all()


def test_weights_written_right_before_the_few_token_kernel(lib):
    # the producer of the packed weights sits directly before the GEMM in the stream; without the
    # stable-weights flag the kernel must not request them before that producer has completed
    m, k, n = 4096, 4096, 4
    p = Problem(43, m, k)
    B = helpers.make_tokens(p.rng, k, n, "int")
    want32, _ = p.oracle(B, use_scale=False)
    d_b = dev(B)
    bits_tile = torch.zeros(m * k // 16, dtype=torch.uint8, device="cuda")
    meta_tile = torch.zeros(m * k // 8, dtype=torch.uint8, device="cuda")
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    for rep in range(5):
        bits_tile.zero_(); meta_tile.zero_()
        _lib.check(lib.onebit_relayout(p.d_bits.data_ptr(), p.d_meta.data_ptr(), p.dialect, m, k, bits_tile.data_ptr(),
                                       meta_tile.data_ptr(), None))
        _lib.check(lib.onebit_matmul_packed(bits_tile.data_ptr(), meta_tile.data_ptr(), None, d_b.data_ptr(), out.data_ptr(),
                                            m, n, k, _lib.OUT_F32, _lib.KERNEL_DECODE, None))
        assert (out.cpu().numpy() == want32).all()
    # with the flag, on weights that are old by then: same result
    _lib.check(lib.onebit_matmul_packed(bits_tile.data_ptr(), meta_tile.data_ptr(), None, d_b.data_ptr(), out.data_ptr(),
                                        m, n, k, _lib.OUT_F32, _lib.KERNEL_DECODE | _lib.KERNEL_STABLE_WEIGHTS, None))
    _lib.check(lib.onebit_check_device_status())
    assert (out.cpu().numpy() == want32).all()


def test_reference_entry_point(lib):
    # the reference's own symbol: CUTLASS-ordered metadata, fp32 D, c ignored, default stream
    m, n, k = 256, 64, 256
    p = Problem(7, m, k, _lib.META_CUTLASS)
    B = helpers.make_tokens(p.rng, k, n, "int")
    want32, _ = p.oracle(B, use_scale=False)
    d_b = dev(B)
    out = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    getattr(lib, _lib.LEGACY_SYMBOL)(p.d_bits.data_ptr(), d_b.data_ptr(), out.data_ptr(), out.data_ptr(), p.d_meta.data_ptr(), m, n, k)
    _lib.check(lib.onebit_check_device_status())
    assert (out.cpu().numpy() == want32).all()


def test_reference_cli_degenerate_fill(lib):
    # the reference CLI's default data: all sign bits 1, metadata 0x4444 everywhere
    # (tests/kernel_test.cu:302-306,398-400): C[i, j] = sum_g B[4g, j] + B[4g + 1, j]
    m, n, k = 128, 32, 256
    a_bits = torch.full((k // 2, m // 8), 0xFF, dtype=torch.uint8, device="cuda")
    e_meta = torch.full((m, k // 16), 0x4444, dtype=torch.int16, device="cuda")
    B = np.random.default_rng(3).integers(-8, 9, size=(k, n)).astype(np.float16)
    d_b = dev(B)
    out = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    _lib.check(lib.onebit_sparse_matmul_ex(a_bits.data_ptr(), d_b.data_ptr(), out.data_ptr(), e_meta.data_ptr(), None,
                                           m, n, k, _lib.OUT_F32, _lib.META_CUTLASS, None, 0, None))
    _lib.check(lib.onebit_check_device_status())
    want = B.astype(np.float32).reshape(k // 4, 4, n)[:, :2].sum(axis=(0, 1))
    assert (out.cpu().numpy() == want[None, :]).all()


def test_python_module_forward(lib):
    import onebitsparsemul_b200 as ob
    rng = np.random.default_rng(21)
    m, k = 256, 384
    dense, scale = helpers.make_weights(rng, m, k)
    w = torch.from_numpy(dense * np.float16(0.5))
    layer = ob.BinaryLinear_2_4(k, m).cuda()
    with pytest.raises(NotImplementedError):
        layer(torch.zeros((k, 8), dtype=torch.float16, device="cuda"))
    layer.pack(w, scale=torch.from_numpy(scale))
    canon, signs, _ = oracle.compress(dense)
    for n in (4, 64):
        B = helpers.make_tokens(rng, k, n, "int")
        want32, _ = oracle.gemm(oracle.pack_bits(signs), oracle.meta_reorder(canon, 0), 0, B, m, scale=scale)
        got = layer(dev(B)).cpu().numpy()
        assert np.allclose(got, want32, rtol=1e-6, atol=1e-6)
        got2 = ob.cuda_binary_mul(layer.packed_binary_sparse, dev(B), layer.meta, scale=layer.scale).cpu().numpy()
        assert (got2 == got).all()


# ---- full benchmark sizes: sampled rows against the oracle + size-independent properties ---------------------

def _gpu_weights(m, k, seed):
    """Random valid 2:4 pattern and signs, generated on the GPU (the benchmark's distributions)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    nib = torch.tensor([0x4, 0x8, 0x9, 0xC, 0xD, 0xE], device="cuda")[torch.randint(0, 6, (m, k // 4), device="cuda", generator=g)]
    sign = (torch.randint(0, 2, (m, k // 4, 2), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    w = torch.zeros((m, k // 4, 4), dtype=torch.float16, device="cuda")
    w.scatter_(2, (nib & 3).unsqueeze(-1), sign[..., 0:1])
    w.scatter_(2, (nib >> 2).unsqueeze(-1), sign[..., 1:2])
    scale = torch.empty(m, device="cuda").uniform_(0.01, 0.1, generator=g).to(torch.float16)
    return w.reshape(m, k), scale


@pytest.mark.parametrize("m,n,k", [(4096, 4096, 4096), (8192, 8192, 8192), (16384, 16384, 16384), (28672, 2048, 8192),
                                   (8192, 2048, 28672), (25600, 25600, 25600), (65536, 8192, 8192)])
def test_full_size_sampled_rows_and_linearity(lib, m, n, k):
    import onebitsparsemul_b200 as ob
    w, scale = _gpu_weights(m, k, seed=m + k)
    pw = ob.pack_weight(w, scale=scale, apply_mask=False, keep_reference=False)
    g = torch.Generator(device="cuda")
    g.manual_seed(n)
    B1 = torch.randint(-8, 9, (k, n), device="cuda", generator=g).to(torch.float16)
    B2 = torch.randint(-8, 9, (k, n), device="cuda", generator=g).to(torch.float16)
    noscale = ob.PackedWeight(m, k, pw.bits_tile, pw.meta_tile, None)
    C1 = ob.matmul_packed(noscale, B1)                       # fp32, integer-exact
    _lib.check(lib.onebit_check_device_status())
    # (1) 128 sampled rows x 512 sampled columns against the oracle, bit for bit
    rows = torch.randperm(m, device="cuda", generator=g)[:128].sort().values
    cols = 512 if n >= 512 else n
    sub = w[rows].cpu().numpy()
    canon, signs, _ = oracle.compress(sub)
    want, _ = oracle.gemm(oracle.pack_bits(signs), oracle.meta_reorder(canon, 0), 0, B1[:, :cols].cpu().numpy(), 128)
    assert (C1[rows][:, :cols].cpu().numpy() == want).all()
    # (2) linearity, exact in integers: W(B1 + B2) = W B1 + W B2
    C2 = ob.matmul_packed(noscale, B2)
    C12 = ob.matmul_packed(noscale, B1 + B2)
    assert torch.equal(C12, C1 + C2)
    del C2, C12
    # (3) the scaled fp16 output is the rounded scaled fp32 output
    C16 = ob.matmul_packed(pw, B1, out_dtype=torch.float16)
    assert torch.equal(C16, (C1 * scale.float()[:, None]).to(torch.float16))
    # (4) the decode kernel agrees with the tensor-memory kernel on the first 16 tokens
    Cd = ob.matmul_packed(noscale, B1[:, :16].contiguous(), kernel=_lib.KERNEL_DECODE)
    assert torch.equal(Cd, C1[:, :16])


# ---- token-major form (nn.Linear convention): y (n, m) = x (n, k) @ W^T + bias ---------------------------------

@pytest.mark.parametrize("m,n,k", [(256, 1, 256), (256, 5, 384), (512, 16, 1024), (256, 17, 256), (512, 200, 640),
                                   (1024, 256, 512), (2048, 1000, 1024), (384, 40, 256), (4096, 2048, 4096)])
def test_token_major_entry_point(lib, m, n, k):
    p = Problem(3 * m + n + k, m, k)
    rng = p.rng
    bias = rng.integers(-4, 5, size=m).astype(np.float16)
    # exact: integer tokens and bias, no scale, fp32 out
    x = helpers.make_tokens(rng, n, k, "int")                     # (n, k): token-major
    want32, _ = p.oracle(np.ascontiguousarray(x.T), use_scale=False)
    want = want32.T + bias.astype(np.float32)[None, :]
    d_x, d_bias = dev(x), dev(bias)
    y = torch.full((n, m), float("nan"), dtype=torch.float32, device="cuda")
    _lib.check(lib.onebit_linear_tokens(p.d_bits_tile.data_ptr(), p.d_meta_tile.data_ptr(), None, d_bias.data_ptr(),
                                        d_x.data_ptr(), y.data_ptr(), m, n, k, _lib.OUT_F32, _lib.KERNEL_AUTO, None))
    _lib.check(lib.onebit_check_device_status())
    assert (y.cpu().numpy() == want).all(), np.abs(y.cpu().numpy() - want).max()
    # tolerance: normal tokens, per-row scale, fp16 out, no bias
    x = helpers.make_tokens(rng, n, k)
    want32, _ = p.oracle(np.ascontiguousarray(x.T), use_scale=True)
    d_x = dev(x)
    y16 = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")
    _lib.check(lib.onebit_linear_tokens(p.d_bits_tile.data_ptr(), p.d_meta_tile.data_ptr(), p.d_scale.data_ptr(), None,
                                        d_x.data_ptr(), y16.data_ptr(), m, n, k, _lib.OUT_F16, _lib.KERNEL_AUTO, None))
    _lib.check(lib.onebit_check_device_status())
    ok, worst = helpers.row_tolerance_ok(y16.cpu().numpy().T, want32)
    assert ok, worst
    # the same bits as the reference-convention call on transposed operands (fp32, integer tokens)
    if m % 256 == 0 and n > 16:
        ref = torch.empty((m, n), dtype=torch.float32, device="cuda")
        xi = dev(helpers.make_tokens(rng, n, k, "int"))
        _lib.check(lib.onebit_matmul_packed(p.d_bits_tile.data_ptr(), p.d_meta_tile.data_ptr(), None, xi.t().contiguous().data_ptr(),
                                            ref.data_ptr(), m, n, k, _lib.OUT_F32, _lib.KERNEL_AUTO, None)) if n % 8 == 0 else None
        if n % 8 == 0:
            _lib.check(lib.onebit_linear_tokens(p.d_bits_tile.data_ptr(), p.d_meta_tile.data_ptr(), None, None, xi.data_ptr(),
                                                y.data_ptr(), m, n, k, _lib.OUT_F32, _lib.KERNEL_AUTO, None))
            assert torch.equal(y, ref.t())


# ---- every kernel variant the dispatcher can pick, forced through the tuning knob -----------------------------

_VARIANT_CHILD = r"""
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1])
import oracle
from onebitsparsemul_b200 import _lib
from tests import helpers
lib = _lib.load()
rng = np.random.default_rng(5)
for (m, n, k) in ((256, 264, 640), (512, 512, 256)):
    dense, scale = helpers.make_weights(rng, m, k)
    canon, signs, _ = oracle.compress(dense)
    bits, meta = oracle.pack_bits(signs), oracle.meta_reorder(canon, 0)
    bt, mt = helpers.tile_order_from_canonical(canon, signs)
    B = helpers.make_tokens(rng, k, n, "int")
    want, _ = oracle.gemm(bits, meta, 0, B, m)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    d_bt, d_mt, d_b = t(bt), t(mt), t(B)
    for out_dtype, code in ((torch.float32, _lib.OUT_F32), (torch.float16, _lib.OUT_F16)):
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
        _lib.check(lib.onebit_matmul_packed(d_bt.data_ptr(), d_mt.data_ptr(), None, d_b.data_ptr(), out.data_ptr(), m, n, k, code, _lib.KERNEL_PREFILL, None))
        _lib.check(lib.onebit_check_device_status())
        assert (out.cpu().numpy() == want.astype(out.cpu().numpy().dtype)).all(), (m, n, k, out_dtype)
print("variant ok")
"""


@pytest.mark.parametrize("variant", ["121", "1121", "1141", "1221", "2", "22", "3", "1"])
def test_every_kernel_variant_exact(variant):
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ONEBIT_PREFILL_VARIANT=variant)
    r = subprocess.run([sys.executable, "-c", _VARIANT_CHILD, root], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "variant ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


# ---- the split-K cluster form of the tensor-memory kernel (tens to hundreds of tokens on small outputs) -----------

_SPLITK_CHILD = r"""
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1])
import oracle
from onebitsparsemul_b200 import _lib
from tests import helpers
lib = _lib.load()
rng = np.random.default_rng(23)
# 20 and 9 weight tiles along k (unequal slices for most splits), ragged token blocks, more than one token block
for (m, n, k) in ((256, 136, 2560), (384, 40, 1152), (128, 264, 1024)):
    dense, scale = helpers.make_weights(rng, m, k)
    canon, signs, _ = oracle.compress(dense)
    bits, meta = oracle.pack_bits(signs), oracle.meta_reorder(canon, 0)
    bt, mt = helpers.tile_order_from_canonical(canon, signs)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    d_bt, d_mt, d_sc = t(bt), t(mt), t(scale)
    B = helpers.make_tokens(rng, k, n, "int")
    want, _ = oracle.gemm(bits, meta, 0, B, m)
    d_b = t(B)
    for out_dtype, code in ((torch.float32, _lib.OUT_F32), (torch.float16, _lib.OUT_F16)):
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
        _lib.check(lib.onebit_matmul_packed(d_bt.data_ptr(), d_mt.data_ptr(), None, d_b.data_ptr(), out.data_ptr(), m, n, k, code, _lib.KERNEL_PREFILL, None))
        _lib.check(lib.onebit_check_device_status())
        assert (out.cpu().numpy() == want.astype(out.cpu().numpy().dtype)).all(), (m, n, k, out_dtype)
    B = helpers.make_tokens(rng, k, n)
    want32, _ = oracle.gemm(bits, meta, 0, B, m, scale=scale)
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    _lib.check(lib.onebit_matmul_packed(d_bt.data_ptr(), d_mt.data_ptr(), d_sc.data_ptr(), t(B).data_ptr(), out.data_ptr(), m, n, k, _lib.OUT_F16, _lib.KERNEL_PREFILL, None))
    _lib.check(lib.onebit_check_device_status())
    ok, worst = helpers.row_tolerance_ok(out.cpu().numpy(), want32)
    assert ok, (m, n, k, worst)
print("split ok")
"""


@pytest.mark.parametrize("split", ["1", "2", "3", "4", "5", "8"])
def test_split_k_cluster_kernel_exact(split):
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ONEBIT_PREFILL_VARIANT="4", ONEBIT_PREFILL_SPLIT=split)
    r = subprocess.run([sys.executable, "-c", _SPLITK_CHILD, root], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "split ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("m,n,k", [(1024, 64, 4096), (4096, 128, 4096), (4096, 256, 4096), (4096, 32, 11008)])
def test_mid_n_shapes_through_the_dispatcher(lib, m, n, k):
    # few output tiles, long k: the dispatcher cuts k over a cluster; exact on integers, in tolerance otherwise
    check_exact_and_tolerance(lib, Problem(m + n + k, m, k), n, _lib.KERNEL_AUTO)


# ---- the persistent CTA-pair kernel walking several output tiles per cluster --------------------------------

_PERSISTENT_CHILD = r"""
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1])
import oracle
from onebitsparsemul_b200 import _lib
from tests import helpers
lib = _lib.load()
rng = np.random.default_rng(11)
# 10 row blocks x 9 token blocks = 90 tiles on 74 clusters; 3 weight tiles along k (an odd count: the last
# pipeline stage is half full); the last token block is ragged
m, n, k = 2560, 2296, 384
dense, scale = helpers.make_weights(rng, m, k)
canon, signs, _ = oracle.compress(dense)
bits, meta = oracle.pack_bits(signs), oracle.meta_reorder(canon, 0)
bt, mt = helpers.tile_order_from_canonical(canon, signs)
B = helpers.make_tokens(rng, k, n, "int")
want, _ = oracle.gemm(bits, meta, 0, B, m)
t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
d_bt, d_mt, d_b = t(bt), t(mt), t(B)
out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
_lib.check(lib.onebit_matmul_packed(d_bt.data_ptr(), d_mt.data_ptr(), None, d_b.data_ptr(), out.data_ptr(), m, n, k, _lib.OUT_F16, _lib.KERNEL_PREFILL, None))
_lib.check(lib.onebit_check_device_status())
assert (out.cpu().numpy() == want.astype(np.float16)).all(), "reference layout"
x = d_b.t().contiguous()
y = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")
_lib.check(lib.onebit_linear_tokens(d_bt.data_ptr(), d_mt.data_ptr(), None, None, x.data_ptr(), y.data_ptr(), m, n, k, _lib.OUT_F16, _lib.KERNEL_PREFILL, None))
_lib.check(lib.onebit_check_device_status())
assert (y.cpu().numpy() == want.astype(np.float16).T).all(), "token-major"
print("persistent ok")
"""


def test_persistent_pair_kernel_many_tiles_exact():
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ONEBIT_PREFILL_VARIANT="3")
    r = subprocess.run([sys.executable, "-c", _PERSISTENT_CHILD, root], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "persistent ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


# ---- the decode kernel with slices longer than its shared-memory ring (weight slots refilled) ----------------

_DECODE_RING_CHILD = r"""
import sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1])
import oracle
from onebitsparsemul_b200 import _lib
from tests import helpers
lib = _lib.load()
rng = np.random.default_rng(13)
m, k = 256, 128 * 37                        # one CTA per row block walks all 37 k tiles: 10 rounds of 4
dense, scale = helpers.make_weights(rng, m, k)
canon, signs, _ = oracle.compress(dense)
bits, meta = oracle.pack_bits(signs), oracle.meta_reorder(canon, 0)
bt, mt = helpers.tile_order_from_canonical(canon, signs)
t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
d_bt, d_mt = t(bt), t(mt)
for n in (1, 4, 5, 7, 8, 12, 16):
    B = helpers.make_tokens(rng, k, n, "int")
    want, _ = oracle.gemm(bits, meta, 0, B, m)
    d_b = t(B)
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    _lib.check(lib.onebit_matmul_packed(d_bt.data_ptr(), d_mt.data_ptr(), None, d_b.data_ptr(), out.data_ptr(), m, n, k, _lib.OUT_F32, _lib.KERNEL_DECODE, None))
    _lib.check(lib.onebit_check_device_status())
    assert (out.cpu().numpy() == want).all(), ("reference layout", n)
    x = d_b.t().contiguous()
    y = torch.full((n, m), float("nan"), dtype=torch.float32, device="cuda")
    _lib.check(lib.onebit_linear_tokens(d_bt.data_ptr(), d_mt.data_ptr(), None, None, x.data_ptr(), y.data_ptr(), m, n, k, _lib.OUT_F32, _lib.KERNEL_DECODE, None))
    _lib.check(lib.onebit_check_device_status())
    assert (y.cpu().numpy() == want.T).all(), ("token-major", n)
print("decode ring ok")
"""


@pytest.mark.parametrize("variant,split", [("1", "1"), ("1", "2"), ("2", "1"), ("2", "2"), ("2", "3"), ("2", "5"), ("2", "7"), ("2", "8")])
def test_decode_kernel_long_slices_exact(variant, split):
    # both few-token kernels (1 = warp-level mma.sp, 2 = tensor memory), forced, with forced K splits: slices longer
    # than the weight ring, an odd number of tiles, unequal slices, every token-staging path, both layouts
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ONEBIT_DECODE_SPLIT=split, ONEBIT_DECODE_VARIANT=variant)
    r = subprocess.run([sys.executable, "-c", _DECODE_RING_CHILD, root], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "decode ring ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


# ---- one GEMM, several destinations (the fused all-gather's epilogue, here with local buffers) ---------------

@pytest.mark.parametrize("m,n,k,n_extra", [(512, 264, 384, 1), (2560, 2296, 256, 3), (256, 8, 128, 7)])
def test_scatter_epilogue_writes_every_destination(m, n, k, n_extra):
    import onebitsparsemul_b200 as ob
    rng = np.random.default_rng(17)
    dense, scale = helpers.make_weights(rng, m, k)
    pw = ob.pack_weight(torch.from_numpy(dense).cuda(), scale=torch.from_numpy(scale).cuda())
    B = torch.from_numpy(helpers.make_tokens(rng, k, n)).cuda()
    want = ob.matmul_packed(pw, B, out_dtype=torch.float16, kernel=_lib.KERNEL_PREFILL)
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    extra = [torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda") for _ in range(n_extra)]
    ob.matmul_scatter(pw, B, out, [e.data_ptr() for e in extra])
    _lib.check(_lib.load().onebit_check_device_status())
    assert torch.equal(out, want)
    for e in extra:
        assert torch.equal(e, want)
