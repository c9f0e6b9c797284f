// The 2:4 magnitude mask of one group of four fp16 weights, stated weight by weight. The kernels (mask.cu, pack.cu)
// compute the same thing two weights per register (pack16.h); tests/host/pack16_check.cpp checks that form against
// this one. Restates mask_creator of the reference
// (onebit_sparse_mul/_semi_structured_conversions.py:286-314: abs, argsort per group of 4, zero the two
// smallest); torch.argsort leaves the order of equal magnitudes unspecified, here the lower index is dropped first.
#pragma once
#include <stdint.h>

// bit t set = weight t of the group is kept. The keys |w| * 4 + t are distinct, so that six comparisons rank the
// group: weight t is kept when at least two keys are smaller than its own.
__device__ __forceinline__ unsigned ob_keep_mask4(const uint16_t* w) {
  const unsigned k0 = (w[0] & 0x7fffu) * 4u, k1 = (w[1] & 0x7fffu) * 4u + 1u;   // |w| of an fp16 orders like its low 15 bits; NaN last
  const unsigned k2 = (w[2] & 0x7fffu) * 4u + 2u, k3 = (w[3] & 0x7fffu) * 4u + 3u;
  const int c01 = k0 < k1, c02 = k0 < k2, c03 = k0 < k3, c12 = k1 < k2, c13 = k1 < k3, c23 = k2 < k3;
  const int r0 = 3 - c01 - c02 - c03, r1 = c01 + 2 - c12 - c13, r2 = c02 + c12 + 1 - c23, r3 = c03 + c13 + c23;
  return (r0 >= 2 ? 1u : 0u) | (r1 >= 2 ? 2u : 0u) | (r2 >= 2 ? 4u : 0u) | (r3 >= 2 ? 8u : 0u);
}

// what the reference's `weight * mask` leaves of a dropped weight: a signed zero, a NaN stays a NaN
__device__ __forceinline__ uint16_t ob_dropped_value(uint16_t w) {
  return ((w & 0x7fffu) > 0x7c00u) ? w : (uint16_t)(w & 0x8000u);
}
