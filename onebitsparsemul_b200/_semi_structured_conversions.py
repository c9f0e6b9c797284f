"""2:4 compress / decompress / mask with the reference's function names, on the GPU.

Mirror of ``onebit_sparse_mul/_semi_structured_conversions.py`` of the reference: the same three
functions with the same argument meaning, checks and error messages; the torch-op chains are
replaced by the pack, mask and unpack kernels of libonebitmul. Tensors given on the CPU are copied
to the current CUDA device and the results copied back.
"""
from __future__ import annotations

import torch

from . import _lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _cuda(t):
    if not torch.cuda.is_available():
        raise _lib.OneBitError("no CUDA device: this library has no CPU path")
    return t if t.is_cuda else t.cuda()


def sparse_semi_structured_from_dense_cutlass(dense):
    """dense (m, k) -> (kept values (m, k/2), meta int16 (m, k/16) in the reference's order).
    Reference: _semi_structured_conversions.py:54-179 (float32 / int8 inputs are not taken here)."""
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    m, k = dense.shape
    codes = {torch.float16: _lib.DENSE_F16, torch.bfloat16: _lib.DENSE_BF16, torch.int32: _lib.DENSE_I32}
    if dense.dtype not in codes:
        raise RuntimeError(f"Invalid datatype {dense.dtype} of dense matrix")
    if m % 32 != 0:
        raise RuntimeError(f"Number of rows of dense matrix {m} must be divisible by 32")
    if k % 16 != 0:
        raise RuntimeError(f"Number of columns of dense matrix {k} must be divisible by 16")
    lib = _lib.load()
    src = _cuda(dense).contiguous()
    with torch.cuda.device(src.device):
        sparse = torch.empty((m, k // 2), dtype=dense.dtype, device=src.device)
        meta = torch.empty((m, k // 16), dtype=torch.int16, device=src.device)
        _lib.check(lib.onebit_pack_from_dense(src.data_ptr(), codes[dense.dtype], m, k, sparse.data_ptr(), None,
                                              meta.data_ptr(), _lib.META_PYTHON, None, None, _stream()))
    return sparse.to(dense.device), meta.to(dense.device)


def sparse_semi_structured_to_dense_cutlass(sparse, meta_reordered):
    """Inverse of the above for values in any dtype (reference: _semi_structured_conversions.py:186-283).
    Index arithmetic only; runs as torch ops on the tensors' device."""
    if sparse.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional sparse tensor, got {sparse.dim()}-dimensional tensor")
    m, kh = sparse.shape
    if meta_reordered.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional meta tensor, got {meta_reordered.dim()}-dimensional tensor")
    if meta_reordered.device != sparse.device:
        raise RuntimeError(f"Expected meta matrix to be on {sparse.device} device, got matrix on {meta_reordered.device} device")
    if meta_reordered.dtype != torch.int16:
        raise RuntimeError(f"Invalid datatype {meta_reordered.dtype} of meta matrix")
    nrows, ncols = meta_reordered.shape
    if nrows != m:
        raise RuntimeError(f"Number of rows of meta matrix {nrows} must be equal to number of columns of spase matrix {m}")
    if ncols * 8 != kh:
        raise RuntimeError(f"Number of columns of sparse matrix {kh} different from the {ncols * 8}, "
                           "expected according to the number of columns of meta matrix")
    dev = sparse.device
    rows = torch.arange(m, device=dev)[:, None]
    cols = torch.arange(ncols, device=dev)[None, :]
    r = rows // 64 * 64 + (rows % 2) * 2 + (rows % 8) // 4 + ((rows % 32) % 4) // 2 * 32 + ((rows % 64) // 8) * 4
    r = r.expand(m, ncols).clone()
    c = cols.expand(m, ncols).clone()
    tr = ((r % 2 == 0) & (c % 2 == 1)).to(torch.int64)
    bl = ((r % 2 == 1) & (c % 2 == 0)).to(torch.int64)
    r, c = r + tr - bl, c - tr + bl
    off = (c // 2) * m * 2 + r * 2 + c % 2
    meta = meta_reordered.reshape(-1)[off.reshape(-1)].reshape(m, ncols).to(torch.int32) & 0xFFFF
    shifts = torch.arange(8, device=dev, dtype=torch.int32) * 2
    e = (meta.unsqueeze(-1) >> shifts) & 3                                   # (m, ncols, 8)
    pos = (torch.arange(ncols, device=dev)[None, :, None] * 16
           + (torch.arange(8, device=dev)[None, None, :] // 2) * 4 + e).reshape(m, kh).to(torch.int64)
    dense = torch.zeros((m, 2 * kh), dtype=sparse.dtype, device=dev)
    dense.scatter_(1, pos, sparse)
    return dense


def mask_creator(tensor):
    """2:4 magnitude mask as float ones/zeros of tensor's shape (reference:
    _semi_structured_conversions.py:286-314). Equal magnitudes: the lower index is dropped first."""
    if tensor.numel() % 4 != 0:
        raise ValueError(f"Tensor of size {tensor.shape} can't be evenly divided into 4 groups")
    if tensor.numel() % 8 != 0:
        raise ValueError("the GPU mask kernel takes element counts divisible by 8")
    lib = _lib.load()
    src = _cuda(tensor.detach()).to(torch.float16).contiguous()
    with torch.cuda.device(src.device):
        mask = torch.empty(src.shape, dtype=torch.uint8, device=src.device)
        _lib.check(lib.onebit_mask24(src.data_ptr(), src.numel(), None, mask.data_ptr(), _stream()))
    return mask.to(torch.float32).to(tensor.device)
