"""K1 (pack), K4 (relayout) and the mask kernel against the oracle and the reference's golden
vectors, through the C ABI. Bit-exact."""
import numpy as np
import pytest
import torch

import oracle
from onebitsparsemul_b200 import _lib
from tests import helpers

pytestmark = pytest.mark.gpu

NP2CODE = {np.dtype(np.float16): _lib.DENSE_F16, np.dtype(np.int32): _lib.DENSE_I32}


@pytest.fixture(scope="module")
def lib():
    assert torch.cuda.is_available()
    return _lib.load()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def gpu_pack(lib, dense_np, code, dialect, tiled=True, want_sparse=True):
    m, k = dense_np.shape
    d = dev(dense_np.view(np.int16) if dense_np.dtype == np.uint16 else dense_np)
    a_bits = torch.full((k // 2, m // 8), 0xAA, dtype=torch.uint8, device="cuda")
    e_meta = torch.full((m, k // 16), -1, dtype=torch.int16, device="cuda")
    sparse = torch.zeros((m, k // 2), dtype=d.dtype, device="cuda") if want_sparse else None
    bits_tile = torch.full((m * k // 16,), 0x55, dtype=torch.uint8, device="cuda") if tiled else None
    meta_tile = torch.full((m * k // 8,), 0x55, dtype=torch.uint8, device="cuda") if tiled else None
    _lib.check(lib.onebit_pack_from_dense(d.data_ptr(), code, m, k, sparse.data_ptr() if want_sparse else None,
                                          a_bits.data_ptr(), e_meta.data_ptr(), dialect,
                                          bits_tile.data_ptr() if tiled else None,
                                          meta_tile.data_ptr() if tiled else None, None))
    torch.cuda.synchronize()
    return (a_bits.cpu().numpy(), e_meta.cpu().numpy(), None if sparse is None else sparse.cpu().numpy(),
            None if bits_tile is None else bits_tile.cpu().numpy(), None if meta_tile is None else meta_tile.cpu().numpy())


@pytest.mark.parametrize("case,code", [("kat", _lib.DENSE_I32), ("f16", _lib.DENSE_F16),
                                       ("bf16", _lib.DENSE_BF16), ("deg", _lib.DENSE_F16)])
def test_pack_matches_reference_golden(lib, golden, case, code):
    dense = golden[f"{case}_dense"] if f"{case}_dense" in golden else golden[f"{case}_dense_bits"]
    a_bits, e_meta, sparse, _, _ = gpu_pack(lib, dense, code, _lib.META_PYTHON, tiled=False)
    assert (a_bits == golden[f"{case}_packed"]).all()
    assert (e_meta == golden[f"{case}_meta"]).all()
    ref_sparse = golden[f"{case}_sparse"] if f"{case}_sparse" in golden else golden[f"{case}_sparse_bits"]
    assert (sparse.view(ref_sparse.dtype) == ref_sparse).all()


@pytest.mark.parametrize("m,k", [(128, 128), (256, 384), (1024, 512), (64, 32), (192, 96), (4096, 4096)])
@pytest.mark.parametrize("dialect", [_lib.META_PYTHON, _lib.META_CUTLASS])
def test_pack_matches_oracle(lib, m, k, dialect):
    rng = np.random.default_rng(m * 7 + k)
    dense, _ = helpers.make_weights(rng, m, k)
    # sprinkle encoder corner cases: extra non-zeros, missing non-zeros, -0.0, NaN, infinities, subnormals
    flat = dense.reshape(-1)
    idx = rng.integers(0, flat.size, size=max(8, flat.size // 50))
    flat[idx] = rng.choice(np.array([0.0, -0.0, 3.0, -2.0, np.nan, np.inf, -np.inf, 6e-8, -6e-8, 3e-5, -3e-5], np.float16), size=idx.size)
    tiled = m % 128 == 0 and k % 128 == 0
    a_bits, e_meta, sparse, bits_tile, meta_tile = gpu_pack(lib, dense, _lib.DENSE_F16, dialect, tiled=tiled)
    canon, signs, osparse = oracle.compress(dense)
    assert (a_bits == oracle.pack_bits(signs)).all()
    assert (e_meta.view(np.uint16) == oracle.meta_reorder(canon, dialect)).all()
    assert (sparse.view(np.uint16) == osparse.view(np.uint16)).all()
    if tiled:
        want_bits, want_meta = helpers.tile_order_from_canonical(canon, signs)
        assert (bits_tile == want_bits).all()
        assert (meta_tile == want_meta).all()


@pytest.mark.parametrize("m,k", [(128, 128), (384, 256), (4096, 4096), (1408, 4096)])
@pytest.mark.parametrize("dialect", [_lib.META_PYTHON, _lib.META_CUTLASS])
def test_relayout_and_unpack(lib, m, k, dialect):
    rng = np.random.default_rng(m + k + dialect)
    dense, scale = helpers.make_weights(rng, m, k)
    canon, signs, _ = oracle.compress(dense)
    a_bits, e_meta = dev(oracle.pack_bits(signs)), dev(oracle.meta_reorder(canon, dialect).view(np.int16))
    bits_tile = torch.zeros(m * k // 16, dtype=torch.uint8, device="cuda")
    meta_tile = torch.zeros(m * k // 8, dtype=torch.uint8, device="cuda")
    _lib.check(lib.onebit_relayout(a_bits.data_ptr(), e_meta.data_ptr(), dialect, m, k, bits_tile.data_ptr(),
                                   meta_tile.data_ptr(), None))
    want_bits, want_meta = helpers.tile_order_from_canonical(canon, signs)
    assert (bits_tile.cpu().numpy() == want_bits).all()
    assert (meta_tile.cpu().numpy() == want_meta).all()
    # tile order -> dense equals the oracle's dequantisation (times the scale)
    out = torch.zeros((m, k), dtype=torch.float16, device="cuda")
    sc = dev(scale)
    _lib.check(lib.onebit_unpack_to_dense(bits_tile.data_ptr(), meta_tile.data_ptr(), sc.data_ptr(), m, k, out.data_ptr(), None))
    deq = oracle.dequant(a_bits.cpu().numpy(), e_meta.cpu().numpy(), dialect, m, k)
    want = (deq.astype(np.float32) * scale.astype(np.float32)[:, None]).astype(np.float16)
    assert (out.cpu().numpy() == want).all()


def test_mask_matches_reference_and_oracle(lib, golden):
    dense = golden["mask_dense"]
    d = dev(dense)
    mask = torch.zeros(dense.shape, dtype=torch.uint8, device="cuda")
    masked = torch.zeros_like(d)
    _lib.check(lib.onebit_mask24(d.data_ptr(), d.numel(), masked.data_ptr(), mask.data_ptr(), None))
    assert (mask.cpu().numpy() == golden["mask_mask"]).all()
    assert (masked.cpu().numpy() == dense * golden["mask_mask"].astype(np.float16)).all()
    # ties and zeros: against the oracle's documented tie rule
    rng = np.random.default_rng(5)
    dense = rng.integers(-3, 4, size=(256, 512)).astype(np.float16)
    d = dev(dense)
    mask = torch.zeros(dense.shape, dtype=torch.uint8, device="cuda")
    _lib.check(lib.onebit_mask24(d.data_ptr(), d.numel(), None, mask.data_ptr(), None))
    assert (mask.cpu().numpy() == oracle.mask24(dense)).all()
    assert (mask.cpu().numpy().reshape(-1, 4).sum(1) == 2).all()


@pytest.mark.parametrize("m,k", [(128, 128), (256, 384), (1024, 4096), (64, 32)])
def test_fused_mask_and_pack_equals_the_two_passes(lib, golden, m, k):
    # unmasked weights with ties, signed zeros, infinities and NaNs: the one-pass kernel must give, byte for byte,
    # what the mask kernel followed by the pack kernel gives -- and the reference's own mask on tie-free data
    rng = np.random.default_rng(m + k)
    dense = (rng.standard_normal((m, k)) * 2).astype(np.float16)
    dense[rng.random((m, k)) < 0.15] = np.float16(0.0)
    dense[rng.random((m, k)) < 0.05] = np.float16(-0.0)
    dense[rng.random((m, k)) < 0.1] = np.float16(1.0)                      # ties
    dense[rng.random((m, k)) < 0.01] = np.float16(np.nan)
    dense[rng.random((m, k)) < 0.01] = np.float16(np.inf)
    dense[rng.random((m, k)) < 0.01] = np.float16(-6e-8)       # subnormals
    dense[rng.random((m, k)) < 0.01] = np.float16(6e-8)
    d = dev(dense)
    tiled = m % 128 == 0 and k % 128 == 0

    def outputs():
        o = dict(masked=torch.zeros_like(d), sparse=torch.zeros((m, k // 2), dtype=torch.float16, device="cuda"),
                 bits=torch.zeros((k // 2, m // 8), dtype=torch.uint8, device="cuda"),
                 meta=torch.zeros((m, k // 16), dtype=torch.int16, device="cuda"))
        if tiled:
            o.update(bits_tile=torch.zeros(m * k // 16, dtype=torch.uint8, device="cuda"),
                     meta_tile=torch.zeros(m * k // 8, dtype=torch.uint8, device="cuda"))
        return o

    ptr = lambda o, name: o[name].data_ptr() if name in o else None
    two, one = outputs(), outputs()
    _lib.check(lib.onebit_mask24(d.data_ptr(), d.numel(), two["masked"].data_ptr(), None, None))
    _lib.check(lib.onebit_pack_from_dense(two["masked"].data_ptr(), _lib.DENSE_F16, m, k, two["sparse"].data_ptr(), two["bits"].data_ptr(),
                                          two["meta"].data_ptr(), _lib.META_PYTHON, ptr(two, "bits_tile"), ptr(two, "meta_tile"), None))
    _lib.check(lib.onebit_mask_pack_from_dense(d.data_ptr(), m, k, one["masked"].data_ptr(), one["sparse"].data_ptr(), one["bits"].data_ptr(),
                                               one["meta"].data_ptr(), _lib.META_PYTHON, ptr(one, "bits_tile"), ptr(one, "meta_tile"), None))
    for name in two:
        a, b = two[name].cpu().numpy(), one[name].cpu().numpy()
        assert (a.view(np.uint8) == b.view(np.uint8)).all(), name
    # without the optional masked copy the packed outputs are the same
    again = outputs()
    _lib.check(lib.onebit_mask_pack_from_dense(d.data_ptr(), m, k, None, None, again["bits"].data_ptr(), again["meta"].data_ptr(),
                                               _lib.META_PYTHON, ptr(again, "bits_tile"), ptr(again, "meta_tile"), None))
    assert torch.equal(again["bits"], one["bits"]) and torch.equal(again["meta"], one["meta"])
    # non-fp16 weights are refused
    assert lib.onebit_mask_pack_from_dense(None, m, k, None, None, None, None, 0, None, None, None) == 2


def test_fused_mask_and_pack_on_the_reference_golden(lib, golden):
    # the reference's mask_creator on tie-free data, then its pack: here in one pass from the unmasked weights
    dense = golden["mask_dense"]
    m, k = dense.shape
    if m % 64 or k % 32:
        pytest.skip("golden mask case is not pack-shaped")
    d = dev(dense)
    bits = torch.zeros((k // 2, m // 8), dtype=torch.uint8, device="cuda")
    meta = torch.zeros((m, k // 16), dtype=torch.int16, device="cuda")
    _lib.check(lib.onebit_mask_pack_from_dense(d.data_ptr(), m, k, None, None, bits.data_ptr(), meta.data_ptr(), _lib.META_PYTHON, None, None, None))
    masked = dense * golden["mask_mask"].astype(np.float16)
    want_bits, want_meta = oracle.pack(masked, oracle.META_PYTHON)
    assert (bits.cpu().numpy() == want_bits).all() and (meta.cpu().numpy() == want_meta).all()


def test_python_api_pack_round_trip(golden):
    import onebitsparsemul_b200 as ob
    dense = torch.from_numpy(golden["f16_dense"])
    sparse, meta = ob.sparse_semi_structured_from_dense_cutlass(dense)
    assert (sparse.numpy() == golden["f16_sparse"]).all() and (meta.numpy() == golden["f16_meta"]).all()
    assert (ob.sparse_semi_structured_to_dense_cutlass(sparse, meta) == dense).all()
    packed = ob.pack_binary(ob.binary_quant(sparse).T.contiguous())
    assert (packed.numpy() == golden["f16_packed"]).all()
    assert (ob.unpack_binary(packed).numpy() == (golden["f16_sparse"].T > 0)).all()
    assert (ob.mask_creator(torch.from_numpy(golden["mask_dense"])).numpy() == golden["mask_mask"]).all()
    # BinaryLinear_2_4.pack on 2:4 input reproduces the reference's stored tensors
    w = torch.from_numpy(golden["f16_dense"]).repeat(1, 2)              # (128, 128)
    layer = ob.BinaryLinear_2_4(128, 128)
    layer.pack(w)
    assert (layer.packed_binary_sparse.cpu().numpy()[:32] == golden["f16_packed"]).all()
    canon_ref = oracle.meta_unreorder(golden["f16_meta"], oracle.META_PYTHON)
    assert (oracle.meta_unreorder(layer.meta.cpu().numpy(), oracle.META_PYTHON)[:, :4] == canon_ref).all()
    assert set(layer.state_dict()) >= {"packed_binary_sparse", "meta", "bits_tile", "meta_tile"}
