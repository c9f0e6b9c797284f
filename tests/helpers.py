"""Shared test helpers: seeded workload generators with the benchmark configs' distributions and a
numpy restatement of the library's tile order (independent of the C headers)."""
from __future__ import annotations

import numpy as np

VALID_NIBBLES = np.array([0x4, 0x8, 0x9, 0xC, 0xD, 0xE], np.uint16)


def make_weights(rng, m, k, scale_dist=True):
    """Dense fp16 W = scale_i * sign * mask with a uniformly random valid 2:4 pattern per group,
    Bernoulli(0.5) signs and a per-row scale U[0.01, 0.1] (the benchmark configs' distributions).
    Returns (dense fp16 (m,k) holding +-1/0, scale fp16 (m,))."""
    nib = VALID_NIBBLES[rng.integers(0, 6, size=(m, k // 4))]
    idx0, idx1 = (nib & 3).astype(np.int64), (nib >> 2).astype(np.int64)
    sign = rng.integers(0, 2, size=(m, k // 4, 2)) * 2 - 1
    dense = np.zeros((m, k // 4, 4), np.float16)
    np.put_along_axis(dense, idx0[..., None], sign[..., 0:1].astype(np.float16), axis=-1)
    np.put_along_axis(dense, idx1[..., None], sign[..., 1:2].astype(np.float16), axis=-1)
    scale = rng.uniform(0.01, 0.1, size=m).astype(np.float16)
    return dense.reshape(m, k), scale


def make_tokens(rng, k, n, kind="normal", sigma=1.0):
    if kind == "int":                          # the reference CLI's exactness fixture: integers in [-8, 8]
        return rng.integers(-8, 9, size=(k, n)).astype(np.float16)
    return (rng.standard_normal((k, n)) * sigma).astype(np.float16)


def tile_order_from_canonical(canon: np.ndarray, signs: np.ndarray):
    """canonical meta (m, k/16) uint16 + signs (m, k/2) 0/1 -> (bits_tile bytes, meta_tile bytes).

    tile (mb, kb) = 128 rows x 128 dense columns, number mb * (k/128) + kb.
    metadata block: 128 lanes x 8 uint16; lane = r0 + 8*c1 + 16*r2, word = 2*c2 + r1 for
      row r = r0 + 8*r1 + 16*r2 and chunk c = c1 + 2*c2 of the tile.
    sign block: row r owns two uint32; kept value v (0..63) -> word v // 32, bit (v%32)//2 + 16*(v%2).
    """
    m, nc = canon.shape
    k = nc * 16
    mt, ktl = m // 128, k // 128
    meta_tile = np.zeros((mt, ktl, 128, 8), np.uint16)
    bits_tile = np.zeros((mt, ktl, 128, 2), np.uint32)
    cb = canon.reshape(mt, 128, ktl, 8)
    sb = signs.reshape(mt, 128, ktl, 64).astype(np.uint32)
    for r in range(128):
        r0, r1, r2 = r & 7, (r >> 3) & 1, r >> 4
        for c in range(8):
            c1, c2 = c & 1, c >> 1
            meta_tile[:, :, r0 + 8 * c1 + 16 * r2, 2 * c2 + r1] = cb[:, r, :, c]
    for v in range(64):
        word, vv = v // 32, v % 32
        bit = vv // 2 + 16 * (vv % 2)
        bits_tile[:, :, :, word] |= sb[:, :, :, v].transpose(0, 2, 1) << np.uint32(bit)
    return bits_tile.reshape(-1).view(np.uint8), meta_tile.reshape(-1).view(np.uint8)


def row_tolerance_ok(got: np.ndarray, want: np.ndarray, rel=1e-2):
    """The path's stated bound: max |err| <= 1e-2 * |row|_inf, per output row."""
    err = np.abs(got.astype(np.float64) - want.astype(np.float64)).max(axis=1)
    bound = rel * np.abs(want.astype(np.float64)).max(axis=1)
    return bool((err <= bound + 1e-12).all()), float((err / np.maximum(bound, 1e-30)).max())
