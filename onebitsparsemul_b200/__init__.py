"""B200-native one-bit 2:4 sparse GEMM: host-side mirror of the reference's Python package.

Same names, argument meaning and error behaviour as ``onebit_sparse_mul/__init__.py`` of the
reference (lines cited per function); underneath, every step is a hand-written sm_100a kernel reached
through the C ABI of ``libonebitmul.so``. torch is used for device memory and streams only.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib
from ._lib import (DENSE_BF16, DENSE_F16, DENSE_I32, KERNEL_AUTO, KERNEL_DECODE, KERNEL_PREFILL, KERNEL_STABLE_WEIGHTS,
                   META_CUTLASS, META_PYTHON, OUT_F16, OUT_F32, OneBitError)
from ._semi_structured_conversions import (mask_creator, sparse_semi_structured_from_dense_cutlass,
                                           sparse_semi_structured_to_dense_cutlass)

__all__ = [
    "cuda_binary_mul", "cuda_binary_mul_", "binary_quant", "pack_binary", "unpack_binary", "dequant_desparse_tile",
    "py_binary_gemm", "BinaryLinear_2_4", "sparse_semi_structured_from_dense_cutlass",
    "sparse_semi_structured_to_dense_cutlass", "mask_creator", "PackedWeight", "pack_weight", "matmul_packed",
    "relayout", "matmul_rows", "matmul_scatter", "matmul_packed_host", "linear_tokens", "replace_linear_layers", "OneBitError",
]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _cuda(t: torch.Tensor) -> torch.Tensor:
    if not torch.cuda.is_available():
        raise OneBitError("no CUDA device: this library has no CPU path")
    return t if t.is_cuda else t.cuda()


def _out_code(dtype) -> int:
    if dtype == torch.float32:
        return OUT_F32
    if dtype == torch.float16:
        return OUT_F16
    raise TypeError(f"C must be float32 or float16, got {dtype}")


def _dense_code(dtype) -> int:
    try:
        return {torch.float16: DENSE_F16, torch.bfloat16: DENSE_BF16, torch.int32: DENSE_I32}[dtype]
    except KeyError:
        raise RuntimeError(f"Invalid datatype {dtype} of dense matrix") from None


# ---- the GEMM entry points (reference: __init__.py:12-19) ------------------------------------------

def cuda_binary_mul_(A, B, C, meta, scale=None):
    """C[m, n] = A_sparse @ B, in place into C (reference ``cuda_binary_mul_``, __init__.py:17-19).

    A: uint8 (k/2, m/8) sign bitfield as ``BinaryLinear_2_4.pack`` produces; B: fp16 (k, n);
    meta: int16 (m, k/16) in the reference packer's order; C: fp32 or fp16 (m, n) on B's device.
    ``scale`` (fp16 (m,), optional) multiplies output rows.
    """
    lib = _lib.load()
    A, B, meta = _cuda(A), _cuda(B), _cuda(meta)
    if B.dtype != torch.float16 or A.dtype != torch.uint8 or meta.dtype != torch.int16:
        raise TypeError("expected A uint8, B float16, meta int16")
    if not C.is_cuda:
        raise OneBitError("C must live on the CUDA device")
    m, k, n = meta.shape[0], B.shape[0], B.shape[1]
    if A.numel() * 16 != m * k or meta.shape[1] * 16 != k or tuple(C.shape) != (m, n):
        raise ValueError(f"shape mismatch: A {tuple(A.shape)}, B {tuple(B.shape)}, meta {tuple(meta.shape)}, C {tuple(C.shape)}")
    A, B, meta = A.contiguous(), B.contiguous(), meta.contiguous()
    if not C.is_contiguous():
        raise ValueError("C must be contiguous")
    if scale is not None:
        scale = _cuda(scale).to(torch.float16).contiguous()
    with torch.cuda.device(B.device):
        need = lib.onebit_workspace_bytes(m, k) if (m % 128 == 0 and k % 128 == 0) else 0
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=B.device)
        _lib.check(lib.onebit_sparse_matmul_ex(_ptr(A), _ptr(B), _ptr(C), _ptr(meta), _ptr(scale), m, n, k,
                                               _out_code(C.dtype), META_PYTHON, _ptr(ws), ws.numel(), _stream()))
    return C


def cuda_binary_mul(A, B, meta, scale=None, out_dtype=torch.float32):
    """Allocates C on B's device and returns it (reference ``cuda_binary_mul``, __init__.py:12-15)."""
    B = _cuda(B)
    C = torch.empty((meta.shape[0], B.shape[1]), dtype=out_dtype, device=B.device)
    return cuda_binary_mul_(A, B, C, meta, scale=scale)


# ---- pack helpers (reference: __init__.py:22-65) -----------------------------------------------------

def binary_quant(tensor):
    """1 where tensor > 0 else 0 (reference __init__.py:22-23)."""
    return torch.where(tensor > 0, torch.tensor(1, device=tensor.device), torch.tensor(0, device=tensor.device))


def pack_binary(tensor):
    """Pack 0/1 values 8 per byte, LSB first, along the last dim (reference __init__.py:25-34)."""
    shape = list(tensor.shape)
    shape[-1] = shape[-1] // 8
    t = tensor.reshape(*shape, 8).to(torch.uint8)
    weights = (1 << torch.arange(8, device=tensor.device, dtype=torch.int32)).to(torch.uint8)
    return (t * weights).sum(dim=-1).to(torch.uint8)


def unpack_binary(packed_tensor):
    """Inverse of pack_binary (reference __init__.py:36-45, there a Python double loop)."""
    shifts = torch.arange(8, device=packed_tensor.device, dtype=torch.uint8)
    bits = (packed_tensor.unsqueeze(-1) >> shifts) & 1
    return bits.reshape(*packed_tensor.shape[:-1], packed_tensor.shape[-1] * 8)


def dequant_desparse_tile(packed_sparse_tile, meta_tile):
    """(rows, k/16) un-transposed sign bytes + reference-ordered meta -> dense {-1,0,+1} (rows, k)
    (reference __init__.py:47-65)."""
    sparse_tile = unpack_binary(packed_sparse_tile)
    sparse_tile = torch.where(sparse_tile == 1, 1, -1).to(torch.int32)
    return sparse_semi_structured_to_dense_cutlass(sparse_tile, meta_tile)


def py_binary_gemm(x, packed_sparse_tensor, sparse_meta):
    """x (t, rows) @ dequant(V) (rows, cols): the reference's check product (__init__.py:67-97).
    Kept for API parity; it is a validation helper, not the hot path."""
    if packed_sparse_tensor.dtype != torch.uint8:
        raise ValueError("packed_sparse_tensor must be `torch.uint8`")
    if packed_sparse_tensor.shape[0] != x.shape[1]:
        raise ValueError("x.shape[1] must equal to packed_sparse_tensor.shape[0], so we can matmul(x, packed_sparse_tensor)")
    if sparse_meta.dtype != torch.int16:
        raise ValueError("Sparse Meta must be `torch.int16`")
    dense_tile = dequant_desparse_tile(packed_sparse_tensor, sparse_meta)
    return torch.matmul(x, dense_tile.to(torch.float16).to(x.device))


# ---- tile-ordered weights: the fast path ---------------------------------------------------------------

class PackedWeight:
    """A weight matrix in this library's streaming order plus its reference-ordered twin.

    ``stable`` says that the packed tensors were complete before the kernel that precedes the next GEMM in
    the stream was launched; the few-token kernel may then request them early
    (``ONEBIT_KERNEL_STABLE_WEIGHTS``). A new object starts out not stable -- the kernel that wrote it may
    be the one right before its first GEMM -- and becomes stable with that first GEMM. Code that rewrites
    the tensors in place must reset the attribute."""

    def __init__(self, m, k, bits_tile, meta_tile, scale=None, packed_binary_sparse=None, meta=None, stable=False):
        self.m, self.k = m, k
        self.bits_tile, self.meta_tile, self.scale = bits_tile, meta_tile, scale
        self.packed_binary_sparse, self.meta = packed_binary_sparse, meta
        self.stable = stable

    # -- persistence (packed_file.py) ---------------------------------------------------------------------
    def save(self, path, bias=None, row0=0, rows_total=None, slab=0, slabs=1):
        """Write the tile-ordered operands (and scale, optional bias) to `path`; see packed_file.py for the
        format. `row0` / `rows_total` / `slab` / `slabs` place a row slab inside a sharded matrix."""
        from . import packed_file
        if self.bits_tile is None:
            raise ValueError("only tile-ordered weights (m, k multiples of 128) can be saved")
        packed_file.save_packed(path, self.bits_tile, self.meta_tile, self.m, self.k, order=packed_file.ORDER_TILE,
                                scale=self.scale, bias=bias, row0=row0, rows_total=rows_total, slab=slab, slabs=slabs)

    @classmethod
    def load(cls, path, device="cuda"):
        """Read a file written by `save` (tile order) or holding reference-ordered operands (those are brought into
        tile order on the GPU). Returns (PackedWeight, bias or None, PackedFileInfo)."""
        from . import packed_file
        info, bits, meta, scale, bias = packed_file.load_packed(path, device)
        if info.order == packed_file.ORDER_TILE:
            return cls(info.m, info.k, bits, meta, scale), bias, info
        pw = relayout(bits, meta, meta_dialect=info.order, scale=scale)
        return pw, bias, info

    def _selector(self, kernel):
        """The kernel selector of the next GEMM on these weights, with the stable-weights flag."""
        flag = KERNEL_STABLE_WEIGHTS if self.stable else 0
        self.stable = True
        return kernel | flag


def pack_weight(weight, scale=None, apply_mask=True, keep_reference=True, meta_dialect=META_PYTHON) -> PackedWeight:
    """Dense (m, k) fp16/bf16/int32 weights -> PackedWeight, entirely on the GPU: 2:4 magnitude mask
    (fp16 only; skip with apply_mask=False when the weights are 2:4 already), compress, encode,
    quantise, bit-pack (the body of reference ``BinaryLinear_2_4.pack``, __init__.py:130-145)."""
    lib = _lib.load()
    w = _cuda(weight).contiguous()
    m, k = w.shape
    dev = w.device
    if apply_mask and w.dtype != torch.float16:
        raise TypeError("the GPU mask takes float16 weights; pass apply_mask=False for pre-masked input")
    with torch.cuda.device(dev):
        tiled = m % 128 == 0 and k % 128 == 0
        bits_tile = torch.empty(m * k // 16, dtype=torch.uint8, device=dev) if tiled else None
        meta_tile = torch.empty(m * k // 8, dtype=torch.uint8, device=dev) if tiled else None
        a_bits = torch.empty((k // 2, m // 8), dtype=torch.uint8, device=dev) if keep_reference else None
        e_meta = torch.empty((m, k // 16), dtype=torch.int16, device=dev) if keep_reference else None
        if apply_mask:                                       # mask, compress, encode, quantise, bit-pack: one pass
            _lib.check(lib.onebit_mask_pack_from_dense(_ptr(w), m, k, None, None, _ptr(a_bits), _ptr(e_meta), meta_dialect,
                                                       _ptr(bits_tile), _ptr(meta_tile), _stream()))
        else:
            _lib.check(lib.onebit_pack_from_dense(_ptr(w), _dense_code(w.dtype), m, k, None, _ptr(a_bits), _ptr(e_meta),
                                                  meta_dialect, _ptr(bits_tile), _ptr(meta_tile), _stream()))
    if scale is not None:
        scale = _cuda(scale).to(torch.float16).contiguous()
    return PackedWeight(m, k, bits_tile, meta_tile, scale, a_bits, e_meta)


def relayout(packed_binary_sparse, meta, meta_dialect=META_PYTHON, scale=None) -> PackedWeight:
    """Reference-ordered operands (what the reference's pack() stores) -> PackedWeight."""
    lib = _lib.load()
    A, meta = _cuda(packed_binary_sparse).contiguous(), _cuda(meta).contiguous()
    m, k = meta.shape[0], meta.shape[1] * 16
    with torch.cuda.device(A.device):
        bits_tile = torch.empty(m * k // 16, dtype=torch.uint8, device=A.device)
        meta_tile = torch.empty(m * k // 8, dtype=torch.uint8, device=A.device)
        _lib.check(lib.onebit_relayout(_ptr(A), _ptr(meta), meta_dialect, m, k, _ptr(bits_tile), _ptr(meta_tile), _stream()))
    if scale is not None:
        scale = _cuda(scale).to(torch.float16).contiguous()
    return PackedWeight(m, k, bits_tile, meta_tile, scale, A, meta)


def matmul_packed(pw: PackedWeight, B, out=None, out_dtype=torch.float32, kernel=KERNEL_AUTO):
    """C (m, n) = pw @ B for B fp16 (k, n) on the weight's device."""
    lib = _lib.load()
    if not B.is_cuda or B.dtype != torch.float16 or B.shape[0] != pw.k:
        raise ValueError("B must be a CUDA float16 tensor of shape (k, n)")
    B = B.contiguous()
    n = B.shape[1]
    if out is None:
        out = torch.empty((pw.m, n), dtype=out_dtype, device=B.device)
    with torch.cuda.device(B.device):
        _lib.check(lib.onebit_matmul_packed(_ptr(pw.bits_tile), _ptr(pw.meta_tile), _ptr(pw.scale), _ptr(B), _ptr(out),
                                            pw.m, n, pw.k, _out_code(out.dtype), pw._selector(kernel), _stream()))
    return out


def linear_tokens(pw: PackedWeight, x, bias=None, out_dtype=torch.float16, kernel=KERNEL_AUTO):
    """y (..., m) = x (..., k) @ W^T (+ bias): the nn.Linear convention, no transposition pass
    (``onebit_linear_tokens``). x: CUDA float16, last dimension k."""
    lib = _lib.load()
    if not x.is_cuda or x.dtype != torch.float16 or x.shape[-1] != pw.k:
        raise ValueError("x must be a CUDA float16 tensor whose last dimension is k")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, pw.k).contiguous()
    n = x2.shape[0]
    y = torch.empty((n, pw.m), dtype=out_dtype, device=x.device)
    if n > 0:
        with torch.cuda.device(x.device):
            _lib.check(lib.onebit_linear_tokens(_ptr(pw.bits_tile), _ptr(pw.meta_tile), _ptr(pw.scale), _ptr(bias), _ptr(x2),
                                                _ptr(y), pw.m, n, pw.k, _out_code(out_dtype), pw._selector(kernel), _stream()))
    return y.reshape(*lead, pw.m)


_host_ws = {}


def matmul_packed_host(pw: PackedWeight, B_host, out_host=None, out_dtype=torch.float16):
    """C = pw @ B for tokens B (k, n) in pinned HOST memory, result into pinned host memory: column
    panels of B travel to the GPU, are multiplied and travel back in an overlapped three-stage pipeline
    (``onebit_matmul_packed_host``). Returns the host tensor; the work is queued asynchronously on the
    current stream of the weight's device, so synchronise that stream before reading the result."""
    lib = _lib.load()
    if B_host.is_cuda or B_host.dtype != torch.float16 or B_host.shape[0] != pw.k or not B_host.is_contiguous():
        raise ValueError("B_host must be a contiguous CPU float16 tensor of shape (k, n)")
    if not B_host.is_pinned():
        raise ValueError("B_host must be pinned (page-locked) host memory")
    n = B_host.shape[1]
    if out_host is None:
        out_host = torch.empty((pw.m, n), dtype=out_dtype).pin_memory()
    if out_host.is_cuda or not out_host.is_pinned() or tuple(out_host.shape) != (pw.m, n) or not out_host.is_contiguous():
        raise ValueError("out_host must be a contiguous pinned CPU tensor of shape (m, n)")
    dev = pw.bits_tile.device
    code = _out_code(out_host.dtype)
    need = lib.onebit_host_workspace_bytes(pw.m, n, pw.k, code)
    ws = _host_ws.get(dev)
    if ws is None or ws.numel() < need:
        ws = _host_ws[dev] = torch.empty(need, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.onebit_matmul_packed_host(_ptr(pw.bits_tile), _ptr(pw.meta_tile), _ptr(pw.scale), B_host.data_ptr(),
                                                 out_host.data_ptr(), pw.m, n, pw.k, code, _ptr(ws), ws.numel(), _stream()))
    return out_host


def matmul_rows(pw: PackedWeight, B, out, row0: int, rows: int, kernel=KERNEL_AUTO):
    """out (rows, n) = pw[row0:row0+rows] @ B: the GEMM on a block of whole 128-row tiles of a packed
    weight (tile order keeps the tiles of a row block contiguous, so this is pointer arithmetic)."""
    lib = _lib.load()
    if row0 % 128 or rows % 128 or row0 + rows > pw.m:
        raise ValueError("row blocks must be whole 128-row tiles inside the weight")
    if not B.is_cuda or B.dtype != torch.float16 or B.shape[0] != pw.k:
        raise ValueError("B must be a CUDA float16 tensor of shape (k, n)")
    B = B.contiguous()
    n = B.shape[1]
    if tuple(out.shape) != (rows, n) or not out.is_contiguous():
        raise ValueError("out must be a contiguous (rows, n) tensor")
    tiles = (row0 // 128) * (pw.k // 128)
    scale_ptr = None if pw.scale is None else pw.scale.data_ptr() + 2 * row0
    with torch.cuda.device(B.device):
        _lib.check(lib.onebit_matmul_packed(pw.bits_tile.data_ptr() + tiles * 1024, pw.meta_tile.data_ptr() + tiles * 2048,
                                            scale_ptr, _ptr(B), _ptr(out), rows, n, pw.k, _out_code(out.dtype),
                                            pw._selector(kernel), _stream()))
    return out


def matmul_scatter(pw: PackedWeight, B, out, extra_ptrs):
    """out (m, n) fp16 = pw @ B, written in the same pass to `out` and to every address in
    `extra_ptrs` (at most 7 integers: device-accessible, 16-byte aligned buffers of out's shape, e.g. this
    rank's row slab inside the peers' copies of C): ``onebit_matmul_packed_scatter``. The caller orders the
    GPUs around the call."""
    import ctypes
    lib = _lib.load()
    if not B.is_cuda or B.dtype != torch.float16 or B.shape[0] != pw.k:
        raise ValueError("B must be a CUDA float16 tensor of shape (k, n)")
    B = B.contiguous()
    n = B.shape[1]
    if tuple(out.shape) != (pw.m, n) or out.dtype != torch.float16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous float16 (m, n) tensor")
    extra = (ctypes.c_void_p * max(1, len(extra_ptrs)))(*[int(p) for p in extra_ptrs])
    with torch.cuda.device(B.device):
        _lib.check(lib.onebit_matmul_packed_scatter(_ptr(pw.bits_tile), _ptr(pw.meta_tile), _ptr(pw.scale), _ptr(B), _ptr(out),
                                                    ctypes.cast(extra, ctypes.c_void_p), len(extra_ptrs), pw.m, n, pw.k, _stream()))
    return out


# ---- the module (reference: __init__.py:101-145) ----------------------------------------------------------

class BinaryLinear_2_4(nn.Module):
    """1-bit 2:4 sparse linear layer (reference ``BinaryLinear_2_4``, __init__.py:101-145).

    Same attributes as the reference (``packed_binary_sparse`` uint8 (in/2, out/8), ``meta`` int16
    (out, in/16), ``vaild``), here registered as buffers together with the tile-ordered operands the
    kernels read, so that ``state_dict`` and ``.to()`` carry them. ``forward(x)`` takes x as the
    kernel does, (in, tokens), and returns (out, tokens), like the reference. ``forward_tokens(x)``
    is the ``nn.Linear`` convention, (..., in) -> (..., out), with the optional bias the reference's
    model-replace demo attaches (tests/python/test_model_replace.py:40-42).
    """

    def __init__(self, infeatures: int, outfeatures: int, out_dtype=torch.float32, bias: bool = False):
        super().__init__()
        if infeatures % 128 != 0 or outfeatures % 128 != 0:
            raise ValueError("`infeatures` and `outfeatures` must be divisible by 128.")
        self.infeatures, self.outfeatures, self.out_dtype = infeatures, outfeatures, out_dtype
        self.register_buffer("packed_binary_sparse", torch.zeros((infeatures // 2, outfeatures // 8), dtype=torch.uint8))
        self.register_buffer("meta", torch.zeros((outfeatures, infeatures // 16), dtype=torch.int16))
        self.register_buffer("bits_tile", torch.zeros(outfeatures * infeatures // 16, dtype=torch.uint8))
        self.register_buffer("meta_tile", torch.zeros(outfeatures * infeatures // 8, dtype=torch.uint8))
        self.register_buffer("scale", torch.ones(outfeatures, dtype=torch.float16))
        self.register_buffer("bias", torch.zeros(outfeatures, dtype=torch.float16) if bias else None)
        self.register_buffer("packed_flag", torch.zeros((), dtype=torch.uint8))     # makes `vaild` survive state_dict
        self.vaild = False                # (sic) the reference's attribute name, __init__.py:117
        self._weights_stable = False      # see PackedWeight.stable; reset whenever the buffers are rewritten

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        self.vaild = bool(self.packed_flag.item())
        self._weights_stable = False

    def _apply(self, fn, *args, **kwargs):
        self._weights_stable = False      # .to() / .cuda() copy the buffers with kernels of the current stream
        return super()._apply(fn, *args, **kwargs)

    def _packed(self):
        # the scale defaults to ones: multiplying by 1 is exact, so an unscaled layer equals the reference's
        pw = PackedWeight(self.outfeatures, self.infeatures, self.bits_tile, self.meta_tile, self.scale,
                          stable=self._weights_stable)
        self._weights_stable = True
        return pw

    def forward(self, x):
        """x: (infeatures, tokens) fp16 on the layer's device -> (outfeatures, tokens)."""
        if not self.vaild:
            raise NotImplementedError("the BinaryLinear")
        return matmul_packed(self._packed(), x, out_dtype=self.out_dtype)

    def forward_tokens(self, x):
        """x: (..., infeatures) -> (..., outfeatures), the nn.Linear convention (plus bias if present).
        Token-major kernels: x is read as it lies and y is written as it lies, nothing is transposed."""
        if not self.vaild:
            raise NotImplementedError("the BinaryLinear")
        y = linear_tokens(self._packed(), x.to(torch.float16), bias=self.bias, out_dtype=torch.float16)
        return y if x.dtype == torch.float16 or not x.dtype.is_floating_point else y.to(x.dtype)

    def pack(self, weight, scale=None, bias=None):
        """weight: (outfeatures, infeatures). Mask to 2:4 by magnitude, compress, quantise, pack."""
        if tuple(weight.shape) != (self.outfeatures, self.infeatures):
            raise ValueError(f"weight must be ({self.outfeatures}, {self.infeatures})")
        pw = pack_weight(weight.to(torch.float16) if weight.dtype == torch.float32 else weight, scale=scale)
        self.packed_binary_sparse, self.meta = pw.packed_binary_sparse, pw.meta
        self.bits_tile, self.meta_tile = pw.bits_tile, pw.meta_tile
        dev = pw.bits_tile.device
        self.scale = pw.scale if pw.scale is not None else torch.ones(self.outfeatures, dtype=torch.float16, device=dev)
        if bias is not None:
            self.bias = bias.detach().to(dev, torch.float16).clone()
        self.packed_flag = torch.ones((), dtype=torch.uint8, device=dev)
        self.vaild = True
        self._weights_stable = False

    def save_packed(self, path):
        """Store this layer's packed operands, scale and bias in one file (packed_file.py); `from_packed_file` is
        the inverse. The reference-ordered twins are not stored: they are an exchange format, not what runs."""
        if not self.vaild:
            raise NotImplementedError("the BinaryLinear")
        self._packed().save(path, bias=self.bias)

    @classmethod
    def from_packed_file(cls, path, device="cuda", out_dtype=torch.float16) -> "BinaryLinear_2_4":
        pw, bias, info = PackedWeight.load(path, device)
        if info.slabs != 1:
            raise ValueError(f"{path} holds slab {info.slab} of {info.slabs}: load it through ShardedBinaryLinear")
        layer = cls(info.k, info.m, out_dtype=out_dtype, bias=bias is not None).to(device)
        layer.bits_tile, layer.meta_tile = pw.bits_tile, pw.meta_tile
        if pw.scale is not None:
            layer.scale = pw.scale
        if bias is not None:
            layer.bias = bias
        layer.packed_flag = torch.ones((), dtype=torch.uint8, device=layer.bits_tile.device)
        layer.vaild = True
        layer._weights_stable = False
        return layer

    @classmethod
    def from_linear(cls, linear: nn.Linear, out_dtype=torch.float16) -> "BinaryLinear_2_4":
        """Quantise an ``nn.Linear``: sign bits of the 2:4-masked weight, per-row scale = mean |w| of the
        kept weights (the scale that minimises the L2 error of a +-scale code), bias carried over."""
        w = linear.weight.detach()
        layer = cls(linear.in_features, linear.out_features, out_dtype=out_dtype, bias=linear.bias is not None)
        wc = w.to("cuda", torch.float16) if not w.is_cuda else w.to(torch.float16)
        mask = mask_creator(wc)
        scale = ((wc.float().abs() * mask).sum(1) / mask.sum(1).clamp(min=1)).to(torch.float16)
        layer = layer.to(wc.device)
        layer.pack(wc, scale=scale, bias=None if linear.bias is None else linear.bias)
        return layer


def replace_linear_layers(model: nn.Module, skip=("lm_head",), min_features: int = 128) -> int:
    """Swap every eligible ``nn.Linear`` of `model` for a packed ``BinaryLinear_2_4`` in place (the flow of
    the reference's tests/python/test_model_replace.py:22-44). A layer is eligible when both feature
    counts are multiples of 128 and its name is not in `skip`. Returns the number of layers replaced.
    The replaced layers answer ``module(x)`` with the nn.Linear convention."""
    replaced = 0
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear) and name not in skip and child.in_features % 128 == 0 \
                and child.out_features % 128 == 0 and min(child.in_features, child.out_features) >= min_features:
            packed = BinaryLinear_2_4.from_linear(child)
            packed.forward = packed.forward_tokens          # nn.Linear calling convention inside a model
            setattr(model, name, packed)
            replaced += 1
        else:
            replaced += replace_linear_layers(child, skip, min_features)
    return replaced
