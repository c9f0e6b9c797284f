// The per-chunk arithmetic of the pack kernel for 16-bit weights (fp16, bf16), two weights per 32-bit register.
//
// A lane of the pack kernel owns one chunk: 16 consecutive weights of one row = 8 registers, weight 2i in the low
// half of register i. Everything below works on both halves of a register at once, and on all four groups of a
// chunk at once where the reference works element by element:
//   * per-weight tests (non-zero, positive, NaN) are additions that carry into bit 15 of each half;
//   * the 2:4 magnitude mask of mask_creator (onebit_sparse_mul/_semi_structured_conversions.py:286-314) ranks a
//     group with six magnitude comparisons, done two at a time as half-wise subtractions; a weight is kept when it
//     wins at least two of its three comparisons, which is one three-input majority per register;
//   * the metadata encoder of sparse_semi_structured_from_dense_cutlass (:54-179; its minimised boolean
//     functions, :133-141) runs on bit planes that hold one bit per group, i.e. once per chunk.
// Plain integer C++, so the same code is checked on the host against the element-wise statement of the rules
// (tests/host/pack16_check.cpp; this header only has to agree with mask24.h and formats.h). The kernels replace the
// per-weight tests by half2 comparisons (FMA pipe) where the data type has them; the integer forms here define
// what those must return.
#pragma once
#include <stdint.h>

#ifndef OB_HD
#ifdef __CUDACC__
#define OB_HD __host__ __device__ __forceinline__
#else
#define OB_HD inline
#endif
#endif

constexpr uint32_t kObSign2 = 0x80008000u, kObMag2 = 0x7fff7fffu;

// a > b for the 15-bit magnitudes in both halves: bit 15 / 31 of the result is CLEAR where a > b (the subtraction
// borrows from the guard bit), SET where a <= b. No borrow crosses the halves.
OB_HD uint32_t ob_le2_raw(uint32_t a, uint32_t b) { return (b | kObSign2) - a; }

// swap the halves of a register
OB_HD uint32_t ob_swap2(uint32_t x) { return (x >> 16) | (x << 16); }

// bit 15 / 31 set where the half is NaN. nan_add = 0x7fff - (largest finite-or-inf magnitude): 0x03ff (fp16), 0x007f (bf16)
OB_HD uint32_t ob_nan2(uint32_t x, uint32_t nan_add2) { return ((x & kObMag2) + nan_add2) & kObSign2; }
// bit 15 / 31 set where the half is not +-0
OB_HD uint32_t ob_nonzero2(uint32_t x) { return ((x & kObMag2) + kObMag2) & kObSign2; }

// The 2:4 magnitude mask of one group, fp16: w0 = weights 0, 1, w1 = weights 2, 3 of the group. ob_keep_group2
// returns bit 15 / 31 of keep0 (weights 0, 1) and keep1 (weights 2, 3) set for the two weights that stay; after
// ob_mask_group2 the two weights of smaller magnitude are what `weight * 0` leaves of them: a signed zero, a NaN
// stays a NaN. Among equal magnitudes the lower index is dropped first (the rule of mask24.h).
OB_HD void ob_keep_group2(uint32_t w0, uint32_t w1, uint32_t& keep0, uint32_t& keep1) {
  const uint32_t m0 = w0 & kObMag2, m1 = w1 & kObMag2;
  // "u beats t" for u < t means |u| > |t| (a tie goes to the higher index). le bits: SET = the lower index loses.
  const uint32_t c1 = ob_le2_raw(m0, m1);                  // low: 0 vs 2, high: 1 vs 3
  const uint32_t c2 = ob_le2_raw(m0, ob_swap2(m1));        // low: 0 vs 3, high: 1 vs 2
  const uint32_t ev = (m0 & 0xffffu) | (m1 << 16), od = (m0 >> 16) | (m1 & 0xffff0000u);
  const uint32_t c3 = ob_le2_raw(ev, od);                  // low: 0 vs 1, high: 2 vs 3
  // weight 0 (low half of w0) is kept when it wins >= 2 of (0v1, 0v2, 0v3): a win is a CLEAR bit.
  // weight 1 (high half of w0): (1v0 = 0 lost = SET bit of 0v1), 1v2, 1v3.
  const uint32_t c3lo = (c3 << 16) | (c3 & 0xffffu);       // 0 vs 1 in both halves
  const uint32_t a3 = c3lo ^ 0x00008000u;                  // low half: SET = 0 won against 1; high half: SET = 1 won
  const uint32_t n1 = ~c1, n2 = ~c2;                       // wins of weights 0 and 1 against 2 and 3 as SET bits
  keep0 = ((n1 & n2) | (n1 & a3) | (n2 & a3)) & kObSign2;
  // weight 2 (low half of w1): 2v0 = SET bit of c1.low, 2v1 = SET bit of c2.high, 2v3 = CLEAR bit of c3.high
  // weight 3 (high half of w1): 3v1 = SET of c1.high, 3v0 = SET of c2.low, 3v2 = SET of c3.high
  const uint32_t c2s = ob_swap2(c2);
  const uint32_t c3hi = (c3 >> 16) | (c3 & 0xffff0000u);   // 2 vs 3 in both halves
  const uint32_t b3 = c3hi ^ 0x00008000u;                  // low: SET = 2 won against 3; high: SET = 3 won
  keep1 = ((c1 & c2s) | (c1 & b3) | (c2s & b3)) & kObSign2;
}

OB_HD void ob_mask_group2(uint32_t& w0, uint32_t& w1) {
  uint32_t keep0, keep1;
  ob_keep_group2(w0, w1, keep0, keep1);
  // kept, or NaN: the whole half passes; else only the sign bit
  const uint32_t pass0 = keep0 | ob_nan2(w0, 0x03ff03ffu), pass1 = keep1 | ob_nan2(w1, 0x03ff03ffu);
  w0 &= ((pass0 >> 15) * 0xffffu) | kObSign2;
  w1 &= ((pass1 >> 15) * 0xffffu) | kObSign2;
}

// The encoder on bit masks of a chunk: M / P bit j set = weight j is non-zero / positive (sign bit clear, not zero,
// not NaN). Returns the canonical metadata word (nibble g = the two 2-bit positions of group g's kept weights);
// s0 / s1: bit 4g set = the first / second kept weight of group g is positive.
OB_HD uint32_t ob_encode_planes(uint32_t M, uint32_t P, uint32_t& s0, uint32_t& s1) {
  constexpr uint32_t g = 0x1111u;                          // one bit per group
  const uint32_t m0 = M & g, m1 = (M >> 1) & g, m3 = (M >> 3) & g;
  const uint32_t b0 = m1 & ~m0, b1 = g & ~(m0 | m1);
  const uint32_t b2 = (m0 & m1) | b1 | m3, b3 = b0 | (g & ~m1);
  const uint32_t p0 = P & g, p1 = (P >> 1) & g, p2 = (P >> 2) & g, p3 = (P >> 3) & g;
  // first kept position = (b1 b0) in {0, 1, 2}, second = (b3 b2) in {1, 2, 3}
  const uint32_t lo01 = (b0 & p1) | (~b0 & p0);
  s0 = ((b1 & p2) | (~b1 & lo01)) & g;
  const uint32_t hi23 = (b2 & p3) | (~b2 & p2);
  s1 = ((b3 & hi23) | (~b3 & p1)) & g;
  return b0 | (b1 << 1) | (b2 << 2) | (b3 << 3);
}

// Encodes one chunk with integer arithmetic only. x[8]: the 16 weights (after the mask, if any).
OB_HD uint32_t ob_encode_chunk16(const uint32_t x[8], uint32_t nan_add2, uint32_t& s0, uint32_t& s1) {
  uint32_t nzg = 0, posg = 0;                              // bits 2i and 16 + 2i: weight 2i, 2i + 1 of the chunk
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t nz = ob_nonzero2(x[i]);
    const uint32_t pos = nz & ~x[i] & ~ob_nan2(x[i], nan_add2);
    nzg |= nz >> (15 - 2 * i);
    posg |= pos >> (15 - 2 * i);
  }
  return ob_encode_planes((nzg | (nzg >> 15)) & 0xffffu, (posg | (posg >> 15)) & 0xffffu, s0, s1);
}

// bits 0, 4, 8, 12 of a plane -> bits 0, 1, 2, 3
OB_HD uint32_t ob_plane_to_nibble(uint32_t s) {
  const uint32_t t = (s | (s >> 3)) & 0x0303u;
  return (t | (t >> 6)) & 0xfu;
}
