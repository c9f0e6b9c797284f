// Storage formats of the one-bit 2:4 sparse weight matrix, written once as index functions and
// shared by every kernel and by the host code.
//
// Vocabulary (m = weight rows / output features, k = dense weight columns):
//   * group   : 4 consecutive dense columns of one row; exactly 2 of them are kept.
//   * nibble  : 4 metadata bits of one group = idx0 | idx1 << 2, idx0 < idx1 the kept positions
//               (reference: onebit_sparse_mul/_semi_structured_conversions.py:150-159).
//   * chunk   : 16 dense columns of one row = 4 groups = one uint16 metadata word, nibble j in
//               bits 4j..4j+3 covering dense columns 16c+4j .. 16c+4j+3.
//   * kept value q of a row (q in [0, k/2)): q = 2*group + t for the t-th kept value of the group;
//               its sign bit is 1 for +1 and 0 for -1 (csrc/warp.h:40-51 of the reference).
//
// Three metadata orders exist for the same canonical matrix Meta[row][chunk]:
//   * OB_META_PYTHON  : the order produced by the reference Python packer
//                       (_semi_structured_conversions.py:21-48; rows shuffled in groups of 64).
//   * OB_META_CUTLASS : the order the reference kernel's E operand expects (CUTLASS reorder_meta
//                       for 2-byte elements, rows shuffled in groups of 32, then
//                       ColumnMajorInterleaved<2>; csrc/threadblock.h:198-199).
//   * tile order      : this library's own order (below), one 2 KiB block per 128x128 tile,
//                       directly copyable into tensor memory for tcgen05.mma.sp.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define OB_HD __host__ __device__ __forceinline__
#else
#define OB_HD inline
#endif

enum ObMetaDialect { OB_META_PYTHON = 0, OB_META_CUTLASS = 1 };
enum ObOutType { OB_OUT_F32 = 0, OB_OUT_F16 = 1 };
enum ObDenseType { OB_DENSE_F16 = 0, OB_DENSE_BF16 = 1, OB_DENSE_I32 = 2 };

// ---- reference-side orders ------------------------------------------------------------------

// Where canonical Meta[row][chunk] goes in a reference-ordered metadata buffer: shuffled row r and
// column c, before the column-pair-major linearisation.
OB_HD void ob_meta_ref_position(int dialect, int64_t row, int64_t chunk, int64_t* r_out, int64_t* c_out) {
  int64_t r;
  if (dialect == OB_META_PYTHON) {
    r = (row / 64) * 64 + (row % 2) * 2 + (row % 8) / 4 + ((row % 4) / 2) * 32 + ((row % 64) / 8) * 4;
  } else {
    r = (row / 32) * 32 + (row % 8) * 4 + (row % 32) / 8;
  }
  int64_t c = chunk;
  // 2x2 block swizzle "from Z to N"
  if ((r % 2 == 0) && (c % 2 == 1)) { r += 1; c -= 1; }
  else if ((r % 2 == 1) && (c % 2 == 0)) { r -= 1; c += 1; }
  *r_out = r;
  *c_out = c;
}

// The same permutation on coordinates inside one 128-row block (both row shuffles stay inside 64 / 32 rows, the
// column swap inside a pair of chunks): unsigned arithmetic, for device code that works tile by tile.
OB_HD void ob_meta_ref_position_local(int dialect, unsigned row, unsigned chunk, unsigned* r_out, unsigned* c_out) {
  unsigned r;
  if (dialect == OB_META_PYTHON) {
    r = (row & ~63u) + (row & 1u) * 2 + ((row >> 2) & 1u) + ((row >> 1) & 1u) * 32 + ((row >> 3) & 7u) * 4;
  } else {
    r = (row & ~31u) + (row & 7u) * 4 + ((row >> 3) & 3u);
  }
  // the 2x2 swap exchanges the low bits of row and column when they differ
  const unsigned x = (r ^ chunk) & 1u;
  *r_out = r ^ x;
  *c_out = chunk ^ x;
}

// Flat uint16 offset of canonical Meta[row][chunk] inside a reference-ordered metadata buffer of
// an (m x k) matrix: column-major, interleaved by 2 columns (nchunks = k/16 is not needed).
OB_HD int64_t ob_meta_ref_offset(int dialect, int64_t m, int64_t row, int64_t chunk) {
  int64_t r, c;
  ob_meta_ref_position(dialect, row, chunk, &r, &c);
  return (c / 2) * (2 * m) + r * 2 + (c % 2);
}

// Row-count granularity each reference order needs.
OB_HD int ob_meta_row_granule(int dialect) { return dialect == OB_META_PYTHON ? 64 : 32; }

// Bit index of sign bit (row, q) inside the reference A bitfield: column-major in m, LSB first
// (byte idx >> 3, bit idx & 7). As a uint8 tensor the bitfield has shape (k/2, m/8).
OB_HD int64_t ob_bits_ref_index(int64_t m, int64_t row, int64_t q) { return q * m + row; }

// ---- tile order (this library) --------------------------------------------------------------
//
// The matrix is cut into tiles of 128 rows x 128 dense columns, stored tile after tile with the
// k index fastest: tile (mb, kb) is number mb * (k/128) + kb.
//
//   sign bits : 1 KiB per tile. Row r (0..127) owns 8 bytes at offset 8*r = two uint32 words;
//               word h covers kept values 32h .. 32h+31 of the tile row. Kept value v of a word
//               sits at bit (v >> 1) + 16 * (v & 1), so that one shift and one logic op turn a
//               word into a pair of fp16 +-1 values (even value in the low half).
//   metadata  : 2 KiB per tile = 128 lanes x 16 bytes. Lane u = r0 + 8*c1 + 16*r2 holds, as
//               uint16 word number 2*c2 + r1, the canonical word of
//                   row   = r0 + 8*r1 + 16*r2          (r0 < 8, r1 < 2, r2 < 8)
//                   chunk = 8*kb + 2*c2 + c1            (c1 < 2, c2 < 4)
//               i.e. each 32-bit column c2 of a lane pairs row r (low half) with row r+8 (high
//               half) for one 16-column chunk. tcgen05.cp.128x128b moves the block unchanged
//               into 4 tensor-memory columns; column c2 then serves the MMA of dense columns
//               32*c2 .. 32*c2+31 of the tile. The same block feeds mma.sp.m16n8k32 directly.
#define OB_TILE_M 128
#define OB_TILE_K 128
#define OB_TILE_BITS_BYTES 1024
#define OB_TILE_META_BYTES 2048

OB_HD int64_t ob_tile_index(int64_t k, int64_t row, int64_t col) {
  return (row / OB_TILE_M) * (k / OB_TILE_K) + (col / OB_TILE_K);
}

// uint16 index (within the whole tile-ordered metadata buffer) of canonical Meta[row][chunk].
OB_HD int64_t ob_meta_tile_offset(int64_t k, int64_t row, int64_t chunk) {
  const int64_t tile = ob_tile_index(k, row, chunk * 16);
  const int r = (int)(row % OB_TILE_M);
  const int c = (int)(chunk % 8);
  const int r0 = r & 7, r1 = (r >> 3) & 1, r2 = r >> 4;
  const int c1 = c & 1, c2 = c >> 1;
  const int lane = r0 + 8 * c1 + 16 * r2;
  return tile * (OB_TILE_META_BYTES / 2) + lane * 8 + 2 * c2 + r1;
}

// Bit index (within the whole tile-ordered sign buffer, LSB-first inside little-endian uint32
// words) of sign bit (row, q).
OB_HD int64_t ob_bits_tile_index(int64_t k, int64_t row, int64_t q) {
  const int64_t tile = ob_tile_index(k, row, q * 2);
  const int r = (int)(row % OB_TILE_M);
  const int v64 = (int)(q % 64);          // kept value inside the tile row
  const int word = v64 >> 5, v = v64 & 31;
  const int bit = (v >> 1) + 16 * (v & 1);
  return tile * (OB_TILE_BITS_BYTES * 8) + (int64_t)r * 64 + word * 32 + bit;
}

// ---- the 2:4 encoder ------------------------------------------------------------------------
// Non-zero flags of a group -> nibble, the reference's minimised boolean functions
// (_semi_structured_conversions.py:133-141), valid for every one of the 16 flag patterns.
OB_HD unsigned ob_encode_group(bool m0, bool m1, bool /*m2*/, bool m3) {
  const bool expr0 = m0 && m1, expr1 = !m0 && m1, expr2 = !m0 && !m1;
  const unsigned bit0 = expr1, bit1 = expr2, bit2 = expr0 || expr2 || m3, bit3 = expr1 || !m1;
  return bit0 | (bit1 << 1) | (bit2 << 2) | (bit3 << 3);
}
