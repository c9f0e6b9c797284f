"""Generate tests/golden/golden.npz by EXECUTING the reference's own Python.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py <path-to-reference-checkout>

The reference package imports its CUDA extension at module import
(onebit_sparse_mul/__init__.py:1), so a stub module is inserted first; nothing of the extension is
called. Everything below is the reference's CPU path:

  * pack  : sparse_semi_structured_from_dense_cutlass -> binary_quant -> .T -> pack_binary, the body
            of BinaryLinear_2_4.pack (onebit_sparse_mul/__init__.py:130-145) after masking
  * mask  : mask_creator (_semi_structured_conversions.py:286-314) on tie-free data
  * dequant / gemm : dequant_desparse_tile and py_binary_gemm (__init__.py:47-97)

The committed .npz is what the tests read; the reference itself is never needed at test time.
"""
import os
import sys
import types

import numpy as np
import torch


def load_reference(path):
    sys.modules.setdefault("onebit_sparse_cuda", types.ModuleType("onebit_sparse_cuda"))
    sys.path.insert(0, path)
    import onebit_sparse_mul as ref  # noqa: E402
    return ref


def random_24(rng, m, k, lo=-10, hi=10):
    """Integer-valued matrix with exactly two non-zeros in every group of 4."""
    w = rng.integers(1, hi + 1, size=(m, k)) * rng.choice([-1, 1], size=(m, k))
    keep = np.zeros((m, k // 4, 4), bool)
    pick = np.argsort(rng.random((m, k // 4, 4)), axis=-1)[..., :2]
    np.put_along_axis(keep, pick, True, axis=-1)
    return (w * keep.reshape(m, k)).astype(np.int64)


def ref_pack(ref, dense_t):
    sparse, meta = ref.sparse_semi_structured_from_dense_cutlass(dense_t)
    signs = ref.binary_quant(sparse)
    packed = ref.pack_binary(signs.T.contiguous())
    packed_rowmajor = ref.pack_binary(signs)          # the un-transposed form py_binary_gemm takes
    return sparse, meta, signs, packed, packed_rowmajor


def bits16(t):
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of the reference checkout>")
    ref = load_reference(sys.argv[1])
    rng = np.random.default_rng(3080)
    out = {}

    # --- case kat: the two rows quoted in the reference's tests/python/test_sparse.py:49-67 -----
    kat = random_24(rng, 128, 32)
    kat[0, :16] = [-7, -10, 0, 0, -9, -10, 0, 0, 0, 0, 7, 2, 7, -10, 0, 0]
    kat[1, :16] = [9, -9, 0, 0, 0, 4, 0, -10, 0, 0, -8, 7, 0, -4, 8, 0]
    d = torch.tensor(kat, dtype=torch.int32)
    sparse, meta, signs, packed, _ = ref_pack(ref, d)
    out["kat_dense"] = kat.astype(np.int32)
    out["kat_sparse"] = sparse.numpy()
    out["kat_meta"] = meta.numpy()
    out["kat_signs"] = signs.numpy().astype(np.uint8)
    out["kat_packed"] = packed.numpy()

    # --- case f16: proper 2:4, fp16 ----------------------------------------------------------------
    w = random_24(rng, 128, 64)
    d = torch.tensor(w, dtype=torch.float16) * 0.125
    sparse, meta, signs, packed, _ = ref_pack(ref, d)
    out["f16_dense"] = d.numpy()
    out["f16_sparse"] = sparse.numpy()
    out["f16_meta"] = meta.numpy()
    out["f16_packed"] = packed.numpy()

    # --- case bf16 (stored as bit patterns) --------------------------------------------------------
    w = random_24(rng, 64, 128)
    d = torch.tensor(w, dtype=torch.bfloat16) * 0.5
    sparse, meta, signs, packed, _ = ref_pack(ref, d)
    out["bf16_dense_bits"] = bits16(d)
    out["bf16_sparse_bits"] = bits16(sparse)
    out["bf16_meta"] = meta.numpy()
    out["bf16_packed"] = packed.numpy()

    # --- case deg: every non-zero pattern, exact zeros, -0.0, NaN, inf, subnormals ------------------
    m, k = 64, 64
    vals = np.array([1.0, -1.0, 0.5, -2.0, 6.1e-5, -6.0e-8, np.inf, -np.inf, np.nan], np.float32)
    dd = vals[rng.integers(0, len(vals), size=(m, k))]
    pattern = rng.integers(0, 16, size=(m, k // 4))
    pattern[0, :16] = np.arange(16)
    for t in range(4):
        dd.reshape(m, k // 4, 4)[..., t][(pattern >> t) & 1 == 0] = 0.0
    negz = rng.random((m, k)) < 0.15
    dd[(dd == 0) & negz] = -0.0
    d = torch.tensor(dd, dtype=torch.float16)
    sparse, meta, signs, packed, _ = ref_pack(ref, d)
    out["deg_dense_bits"] = bits16(d)
    out["deg_sparse_bits"] = bits16(sparse)
    out["deg_meta"] = meta.numpy()
    out["deg_packed"] = packed.numpy()

    # --- mask_creator on tie-free magnitudes -------------------------------------------------------
    m, k = 64, 64
    mags = (rng.permutation(m * k).reshape(m, k) % 2000 + 1).astype(np.float32)
    for g in mags.reshape(-1, 4):             # make each group tie-free
        while len(set(g.tolist())) < 4:
            g += rng.integers(0, 4, size=4)
    d = torch.tensor(mags * rng.choice([-1, 1], size=(m, k)), dtype=torch.float16)
    assert all(len(set(abs(g).tolist())) == 4 for g in d.numpy().reshape(-1, 4))
    out["mask_dense"] = d.numpy()
    out["mask_mask"] = ref.mask_creator(d).numpy().astype(np.uint8)

    # --- dequant + CPU GEMM -------------------------------------------------------------------------
    # V (r x c) is 2:4 along c. dequant_desparse_tile takes the un-transposed packing of its signs.
    r, c = 64, 64
    w = random_24(rng, r, c)
    d = torch.tensor(w, dtype=torch.float16)
    sparse, meta, signs, packed, packed_rm = ref_pack(ref, d)
    dense_pm1 = ref.dequant_desparse_tile(packed_rm, meta)                 # (r, c) in {-1,0,1}
    out["gemm_dense"] = d.numpy()
    out["gemm_meta"] = meta.numpy()
    out["gemm_packed"] = packed.numpy()
    out["gemm_dequant"] = dense_pm1.numpy().astype(np.int8)
    # the reference's CPU GEMM, literally: x (t x r) @ dequant(V) (r x c)
    x = torch.tensor(rng.integers(-8, 9, size=(16, r)), dtype=torch.float16)
    out["gemm_x"] = x.numpy()
    out["gemm_py_binary_gemm"] = ref.py_binary_gemm(x, packed_rm, meta).numpy()
    # the product the GPU kernel computes, with the same arithmetic call py_binary_gemm makes
    # (torch.matmul on fp16, __init__.py:95-96): dequant(V) (r x c) @ B (c x n). Integer B keeps every
    # partial sum exact, as the reference CLI's fixture does (tests/kernel_test.cu:321-332).
    B = torch.tensor(rng.integers(-8, 9, size=(c, 24)), dtype=torch.float16)
    out["gemm_B_int"] = B.numpy()
    out["gemm_C_int"] = torch.matmul(dense_pm1.to(torch.float16), B).numpy()
    Bn = torch.tensor(rng.standard_normal((c, 24)), dtype=torch.float16)
    out["gemm_B_normal"] = Bn.numpy()
    out["gemm_C_normal_f32"] = torch.matmul(dense_pm1.to(torch.float32), Bn.to(torch.float32)).numpy()

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
