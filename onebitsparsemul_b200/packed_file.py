"""On-disk format for packed one-bit 2:4 weights.

The reference keeps its pack output -- ``packed_binary_sparse`` and ``meta`` of ``BinaryLinear_2_4.pack``
(onebit_sparse_mul/__init__.py:130-145) -- in plain attributes and has no way to store it. This module is
that missing piece for the operands the kernels here stream: one file holds one row slab of one weight
matrix, so that a row-sharded layer is a set of files and every rank reads only its own.

File layout (little endian, every section starts on a 256-byte boundary):

    offset 0    header, 256 bytes
        0   8s   magic  b"OB24PACK"
        8   I    format version (1)
        12  I    payload order: 2 = tile order (what the GEMM kernels read), 0 / 1 = reference order with the
                 Python / CUTLASS metadata shuffle (the exchange format of the reference packer)
        16  Q    m      rows in this file (a multiple of 128 for tile order)
        24  Q    k      dense columns
        32  Q    row0   first row of this slab inside the whole matrix
        40  Q    rows_total   rows of the whole matrix
        48  I    slab index,  52  I  slab count
        56  I    scale dtype: 0 = none, 1 = float16 (m values)
        60  I    bias dtype:  0 = none, 1 = float16 (m values)
        64  Q    bytes of sign bits,  72  Q  bytes of metadata,  80  Q  bytes of scale,  88  Q  bytes of bias
        96  I    CRC-32 of the four payload sections in file order (padding excluded)
        100 ..   zero
    sign bits | metadata | scale | bias

Tile order is position independent along rows: the tiles of a 128-row block are contiguous, so a slab of whole
128-row blocks packed on its own equals the same rows cut out of a pack of the whole matrix.
"""
from __future__ import annotations

import os
import struct
import zlib
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

MAGIC = b"OB24PACK"
VERSION = 1
ORDER_PYTHON, ORDER_CUTLASS, ORDER_TILE = 0, 1, 2
_HEADER = struct.Struct("<8sIIQQQQIIIIQQQQI")
_ALIGN = 256


class PackedFileError(ValueError):
    """The file is not a packed-weight file of this format, or it is damaged."""


@dataclass
class PackedFileInfo:
    order: int
    m: int
    k: int
    row0: int
    rows_total: int
    slab: int
    slabs: int
    has_scale: bool
    has_bias: bool


def _pad(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


def _bytes(t: Optional[torch.Tensor]) -> bytes:
    if t is None:
        return b""
    return t.detach().contiguous().cpu().numpy().tobytes()


def slab_path(directory: str, name: str, slab: int, slabs: int) -> str:
    """File of slab `slab` of `slabs` of the layer called `name`."""
    return os.path.join(directory, f"{name}.slab{slab:03d}of{slabs:03d}.ob24")


def save_packed(path: str, bits: torch.Tensor, meta: torch.Tensor, m: int, k: int, *, order: int = ORDER_TILE,
                scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, row0: int = 0,
                rows_total: Optional[int] = None, slab: int = 0, slabs: int = 1) -> None:
    """Write one slab. `bits` / `meta` are the uint8 sign bits and the metadata (uint8 for tile order, int16 for
    the reference orders) exactly as the kernels or the reference packer hold them."""
    if order not in (ORDER_PYTHON, ORDER_CUTLASS, ORDER_TILE):
        raise ValueError(f"unknown payload order {order}")
    if m <= 0 or k <= 0 or k % 16 != 0 or (order == ORDER_TILE and (m % 128 or k % 128)):
        raise ValueError(f"shape ({m}, {k}) cannot be stored in order {order}")
    rows_total = m if rows_total is None else rows_total
    sections = [_bytes(bits), _bytes(meta),
                _bytes(None if scale is None else scale.to(torch.float16)), _bytes(None if bias is None else bias.to(torch.float16))]
    if len(sections[0]) != m * k // 16 or len(sections[1]) != m * k // 8:
        raise ValueError(f"sign bits / metadata of {len(sections[0])} / {len(sections[1])} bytes do not belong to a ({m}, {k}) matrix")
    for sec, what in ((sections[2], "scale"), (sections[3], "bias")):
        if sec and len(sec) != 2 * m:
            raise ValueError(f"{what} must have one float16 per row")
    crc = 0
    for sec in sections:
        crc = zlib.crc32(sec, crc)
    header = _HEADER.pack(MAGIC, VERSION, order, m, k, row0, rows_total, slab, slabs, 1 if sections[2] else 0,
                          1 if sections[3] else 0, *[len(s) for s in sections], crc & 0xFFFFFFFF)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(header.ljust(_ALIGN, b"\0"))
        for sec in sections:
            f.write(sec)
            f.write(b"\0" * (_pad(len(sec)) - len(sec)))
    os.replace(tmp, path)                                  # a reader never sees a half-written file


def read_header(path: str) -> PackedFileInfo:
    with open(path, "rb") as f:
        raw = f.read(_ALIGN)
    return _parse_header(raw, path)[0]


def _parse_header(raw: bytes, path: str):
    if len(raw) < _ALIGN or raw[:8] != MAGIC:
        raise PackedFileError(f"{path}: not a packed one-bit weight file")
    (_, version, order, m, k, row0, rows_total, slab, slabs, scale_t, bias_t, nb, nm, ns, nbias, crc) = _HEADER.unpack(raw[:_HEADER.size])
    if version != VERSION:
        raise PackedFileError(f"{path}: format version {version}, this library reads version {VERSION}")
    if order not in (ORDER_PYTHON, ORDER_CUTLASS, ORDER_TILE) or nb != m * k // 16 or nm != m * k // 8 \
            or ns != (2 * m if scale_t else 0) or nbias != (2 * m if bias_t else 0) or row0 + m > rows_total or slab >= slabs:
        raise PackedFileError(f"{path}: inconsistent header")
    info = PackedFileInfo(order, m, k, row0, rows_total, slab, slabs, bool(scale_t), bool(bias_t))
    return info, (nb, nm, ns, nbias), crc


def load_packed(path: str, device="cpu", verify: bool = True):
    """Read one slab. Returns (info, bits, meta, scale, bias) as tensors on `device`; metadata is uint8 for tile
    order and int16 (m, k/16) for the reference orders, sign bits uint8 (flat for tile order, (k/2, m/8) else)."""
    with open(path, "rb") as f:
        raw = f.read()
    info, sizes, crc = _parse_header(raw, path)
    out, off, check = [], _ALIGN, 0
    for n in sizes:
        if off + n > len(raw):
            raise PackedFileError(f"{path}: truncated")
        sec = raw[off:off + n]
        check = zlib.crc32(sec, check)
        out.append(sec)
        off += _pad(n)
    if verify and (check & 0xFFFFFFFF) != crc:
        raise PackedFileError(f"{path}: checksum mismatch (the file is damaged)")
    bits = torch.from_numpy(np.frombuffer(out[0], np.uint8).copy())
    if info.order == ORDER_TILE:
        meta = torch.from_numpy(np.frombuffer(out[1], np.uint8).copy())
    else:
        bits = bits.reshape(info.k // 2, info.m // 8)
        meta = torch.from_numpy(np.frombuffer(out[1], np.int16).copy()).reshape(info.m, info.k // 16)
    scale = torch.from_numpy(np.frombuffer(out[2], np.float16).copy()) if info.has_scale else None
    bias = torch.from_numpy(np.frombuffer(out[3], np.float16).copy()) if info.has_bias else None
    to = lambda t: None if t is None else t.to(device)
    return info, to(bits), to(meta), to(scale), to(bias)
