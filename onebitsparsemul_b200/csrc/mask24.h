// The 2:4 magnitude mask of one group of four fp16 weights, shared by the stand-alone mask kernel (mask.cu) and
// the pack kernel's fused form (pack.cu). Restates mask_creator of the reference
// (onebit_sparse_mul/_semi_structured_conversions.py:286-314: abs, argsort per group of 4, zero the two
// smallest); torch.argsort leaves the order of equal magnitudes unspecified, here the lower index is dropped first.
#pragma once
#include <stdint.h>

// bit t set = weight t of the group is kept
__device__ __forceinline__ unsigned ob_keep_mask4(const uint16_t* w) {
  unsigned keep = 0;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const unsigned at = w[t] & 0x7fffu;       // |w| of an fp16 orders like its low 15 bits; NaN last
    int rank = 0;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const unsigned au = w[u] & 0x7fffu;
      rank += (au < at) || (au == at && u < t);
    }
    keep |= (rank >= 2 ? 1u : 0u) << t;
  }
  return keep;
}

// what the reference's `weight * mask` leaves of a dropped weight: a signed zero, a NaN stays a NaN
__device__ __forceinline__ uint16_t ob_dropped_value(uint16_t w) {
  return ((w & 0x7fffu) > 0x7c00u) ? w : (uint16_t)(w & 0x8000u);
}
