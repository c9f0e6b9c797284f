"""The CPU oracle against the reference's golden vectors (CPU only)."""
import numpy as np
import pytest

import oracle


def test_kat_rows_from_reference_docstring(golden):
    # tests/python/test_sparse.py:49-67 of the reference quotes these rows and their packed form.
    row0 = np.array([-7, -10, 0, 0, -9, -10, 0, 0, 0, 0, 7, 2, 7, -10, 0, 0], np.int32)
    row1 = np.array([9, -9, 0, 0, 0, 4, 0, -10, 0, 0, -8, 7, 0, -4, 8, 0], np.int32)
    dense = golden["kat_dense"]
    assert (dense[0, :16] == row0).all() and (dense[1, :16] == row1).all()
    canon, signs, sparse = oracle.compress(dense)
    assert sparse[0, :8].tolist() == [-7, -10, -9, -10, 7, 2, 7, -10]
    assert sparse[1, :8].tolist() == [9, -9, 4, -10, -8, 7, -4, 8]
    assert signs[0, :8].tolist() == [0, 0, 0, 0, 1, 1, 1, 0]
    assert signs[1, :8].tolist() == [1, 0, 1, 0, 0, 1, 0, 1]
    assert np.packbits(signs[0, :8], bitorder="little")[0] == 112
    assert np.packbits(signs[1, :8], bitorder="little")[0] == 165
    assert canon[0, 0] == 20036 == 0x4E44
    # row 0, chunk 0 keeps its place under the Python shuffle, as the docstring's meta[0] shows
    assert oracle.meta_reorder(canon, oracle.META_PYTHON)[0, 0] == 20036


@pytest.mark.parametrize("case,code", [("kat", oracle.DENSE_I32), ("f16", oracle.DENSE_F16),
                                       ("bf16", oracle.DENSE_BF16), ("deg", oracle.DENSE_F16)])
def test_pack_bit_exact_against_reference(golden, case, code):
    dense = golden[f"{case}_dense"] if f"{case}_dense" in golden else golden[f"{case}_dense_bits"]
    canon, signs, sparse = oracle.compress(dense, code)
    ref_sparse = golden[f"{case}_sparse"] if f"{case}_sparse" in golden else golden[f"{case}_sparse_bits"]
    assert (sparse.view(np.uint16 if sparse.itemsize == 2 else np.int32)
            == ref_sparse.view(np.uint16 if ref_sparse.itemsize == 2 else np.int32)).all()
    meta = oracle.meta_reorder(canon, oracle.META_PYTHON).view(np.int16)
    assert (meta == golden[f"{case}_meta"]).all()
    assert (oracle.pack_bits(signs) == golden[f"{case}_packed"]).all()
    packed, meta2 = oracle.pack(dense, oracle.META_PYTHON, code)
    assert (packed == golden[f"{case}_packed"]).all() and (meta2 == golden[f"{case}_meta"]).all()


def test_encoder_truth_table():
    # all 16 non-zero patterns (_semi_structured_conversions.py:99-124)
    expect = {0b0011: 0x4, 0b0111: 0x4, 0b1011: 0x4, 0b1111: 0x4, 0b0101: 0x8, 0b0001: 0x8,
              0b0110: 0x9, 0b0010: 0x9, 0b1001: 0xC, 0b1101: 0xC, 0b1010: 0xD, 0b1110: 0xD,
              0b1100: 0xE, 0b0100: 0xE, 0b1000: 0xE, 0b0000: 0xE}
    dense = np.zeros((64, 64), np.float16)
    for p in range(16):                      # bit t of p = "element t is non-zero"
        for t in range(4):
            dense[0, 4 * p + t] = 1.0 if (p >> t) & 1 else 0.0
    canon, _, _ = oracle.compress(dense)
    for p in range(16):
        assert (canon[0, p // 4] >> (4 * (p % 4))) & 0xF == expect[p], p


@pytest.mark.parametrize("dialect,gran", [(oracle.META_PYTHON, 64), (oracle.META_CUTLASS, 32)])
def test_meta_orders_are_permutations(dialect, gran):
    m, nc = 3 * gran, 6
    canon = np.arange(m * nc, dtype=np.uint16).reshape(m, nc)
    out = oracle.meta_reorder(canon, dialect)
    assert sorted(out.ravel().tolist()) == list(range(m * nc))
    assert (oracle.meta_unreorder(out, dialect) == canon).all()


def test_cutlass_order_first_rows():
    # CUTLASS reorder_meta sends rows 0..15 of a 32-row group to 0,4,8,... and 1,5,9,...
    m, nc = 32, 2
    canon = np.zeros((m, nc), np.uint16)
    canon[:, 0] = np.arange(m) + 1
    out = oracle.meta_reorder(canon, oracle.META_CUTLASS).ravel()
    dest_rows = [(r % 8) * 4 + r // 8 for r in range(m)]
    for r in range(m):
        rr, cc = dest_rows[r], 0
        if rr % 2 == 1:
            rr, cc = rr - 1, 1
        assert out[(cc // 2) * 2 * m + rr * 2 + cc % 2] == r + 1


def test_dequant_and_gemm_against_reference_cpu_path(golden):
    packed, meta = golden["gemm_packed"], golden["gemm_meta"]
    m, k = golden["gemm_dense"].shape
    deq = oracle.dequant(packed, meta, oracle.META_PYTHON, m, k)
    assert (deq == golden["gemm_dequant"]).all()
    assert (deq == np.sign(golden["gemm_dense"].astype(np.float32)).astype(np.int8)).all()
    # py_binary_gemm literally: x @ dequant(V)
    x = golden["gemm_x"].astype(np.float32)
    assert (x @ deq.astype(np.float32) == golden["gemm_py_binary_gemm"].astype(np.float32)).all()
    # the kernel's product, integer fixture: exact
    c32, c16 = oracle.gemm(packed, meta, oracle.META_PYTHON, golden["gemm_B_int"], m)
    assert (c32 == golden["gemm_C_int"].astype(np.float32)).all()
    assert (c16 == golden["gemm_C_int"]).all()
    # normal B: within the stated tolerance of the path, 1e-2 * |row|_inf
    c32, _ = oracle.gemm(packed, meta, oracle.META_PYTHON, golden["gemm_B_normal"], m)
    ref = golden["gemm_C_normal_f32"]
    assert (np.abs(c32 - ref).max(axis=1) <= 1e-2 * np.abs(ref).max(axis=1)).all()


def test_gemm_dialects_agree_and_scale():
    rng = np.random.default_rng(1)
    m, k, n = 128, 96, 5
    dense = golden_like_dense(rng, m, k)
    canon, signs, _ = oracle.compress(dense)
    bits = oracle.pack_bits(signs)
    B = rng.standard_normal((k, n)).astype(np.float16)
    scale = rng.uniform(0.01, 0.1, m).astype(np.float16)
    outs = []
    for d in (oracle.META_PYTHON, oracle.META_CUTLASS):
        outs.append(oracle.gemm(bits, oracle.meta_reorder(canon, d), d, B, m, scale=scale))
    assert (outs[0][0] == outs[1][0]).all()
    want = (np.sign(dense.astype(np.float32)) @ B.astype(np.float32)) * scale.astype(np.float32)[:, None]
    assert np.allclose(outs[0][0], want, rtol=1e-4, atol=1e-4)
    assert (outs[0][1] == outs[0][0].astype(np.float16)).all()      # RNE fp16 rounding


def golden_like_dense(rng, m, k):
    w = rng.integers(1, 9, size=(m, k)) * rng.choice([-1, 1], size=(m, k))
    keep = np.zeros((m, k // 4, 4), bool)
    np.put_along_axis(keep, np.argsort(rng.random((m, k // 4, 4)), axis=-1)[..., :2], True, axis=-1)
    return (w * keep.reshape(m, k)).astype(np.float16)


def test_fp16_rounding_matches_numpy():
    rng = np.random.default_rng(2)
    vals = np.concatenate([rng.standard_normal(4096) * s for s in (1e-8, 1e-5, 1e-3, 1, 300, 7e4)]).astype(np.float32)
    vals = np.concatenate([vals, np.array([65504, 65519.99, 65520, 2 ** -24, 2 ** -25, 1.5 * 2 ** -25, 0, -0.0], np.float32)])
    m = 128
    n = len(vals) // m
    vals = vals[: m * n]
    # one-hot weights turn the GEMM into a copy of B rows: row i keeps dense column 4*i... use k = 4m
    k = 4 * m
    dense = np.zeros((m, k), np.float16)
    for i in range(m):
        dense[i, 4 * i] = 1.0
        dense[i, 4 * i + 1] = 1.0
    canon, signs, _ = oracle.compress(dense)
    B = np.zeros((k, n), np.float16)
    # fp32 values must come out of the accumulator, so feed halves whose sum is the fp32 value
    with np.errstate(over="ignore"):
        hi = vals.reshape(m, n).astype(np.float16)
    lo = (vals.reshape(m, n) - hi.astype(np.float32)).astype(np.float16)
    hi[~np.isfinite(hi)] = 0
    lo[~np.isfinite(lo)] = 0
    B[0::4][:m] = hi
    B[1::4][:m] = lo
    c32, c16 = oracle.gemm(oracle.pack_bits(signs), oracle.meta_reorder(canon, 0), 0, B, m)
    assert (c16 == c32.astype(np.float16)).all()


def test_mask24_against_reference(golden):
    assert (oracle.mask24(golden["mask_dense"]) == golden["mask_mask"]).all()


def test_gemm_against_the_references_own_host_gemm():
    """The oracle's GEMM against the reference's host check GEMM itself -- the CUTLASS template its CLI instantiates
    (tests/kernel_test.cu:441-456), compiled from the CUTLASS headers on this machine into oracle/_ref/ -- on the same
    seeded operands: integer tokens, so the weighted checksum of the fp32 result must agree exactly."""
    from oracle import build_ref
    if build_ref.build() is None:
        pytest.skip("no CUTLASS copy with host reference utilities on this machine")
    m, n, k = 128, 64, 256
    seconds, gflops, checksum = build_ref.run(m, n, k, seed=11)
    A, B = build_ref.inputs(m, n, k, seed=11)
    canon, signs, _ = oracle.compress(A)
    c32, _ = oracle.gemm(oracle.pack_bits(signs), oracle.meta_reorder(canon, oracle.META_CUTLASS), oracle.META_CUTLASS, B, m)
    weights = (np.arange(m * n) % 7 + 1).astype(np.float64)
    assert float((c32.reshape(-1).astype(np.float64) * weights).sum()) == checksum
    assert (c32 == A.astype(np.float32) @ B.astype(np.float32)).all()


def test_bench_reference_arm_prints_one_json_line():
    # the reference arm of bench.py (the oracle port on the host cores): exactly one line on standard output, a JSON
    # object with the contract's keys, even when something else writes to file descriptor 1 while it runs
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--size", "512", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, cwd=root, env=dict(os.environ, NCCL_DEBUG="VERSION"))
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.splitlines()
    assert len(lines) == 1, r.stdout[:2000]
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["value"] > 0
    for key in ("metric", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] == "port"
