// Magnitude 2:4 mask: in every group of 4 consecutive weights drop the two smallest |w|.
// Replaces mask_creator (onebit_sparse_mul/_semi_structured_conversions.py:286-314: abs, argsort per
// group of 4, scatter zeros), the slowest step of the reference's pack(). torch.argsort leaves the
// order of equal magnitudes unspecified; here the lower index is dropped first. One thread per 8
// weights (two groups, one 16-byte load); HBM-bound.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "mask24.h"

namespace {

__global__ void __launch_bounds__(256) ob_mask24_kernel(const uint4* __restrict__ dense, int64_t vecs,
                                                        uint4* __restrict__ masked, uint2* __restrict__ mask) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= vecs) return;
  uint4 v = __ldg(dense + i);
  uint16_t* w = reinterpret_cast<uint16_t*>(&v);
  const unsigned keep = ob_keep_mask4(w) | (ob_keep_mask4(w + 4) << 4);
  if (mask) {
    uint2 mk;
    uint8_t* mb = reinterpret_cast<uint8_t*>(&mk);
#pragma unroll
    for (int t = 0; t < 8; ++t) mb[t] = (keep >> t) & 1u;
    mask[i] = mk;
  }
  if (masked) {
    // the reference multiplies by the 0/1 mask: a dropped weight becomes a signed zero, a kept NaN stays
#pragma unroll
    for (int t = 0; t < 8; ++t)
      if (!((keep >> t) & 1u)) w[t] = ob_dropped_value(w[t]);
    masked[i] = v;
  }
}

}  // namespace

namespace ob {

cudaError_t launch_mask24(const void* dense_f16, int64_t count, void* masked_f16, void* mask_u8, cudaStream_t stream) {
  const int64_t vecs = count / 8;
  if (vecs == 0) return cudaSuccess;
  ob_mask24_kernel<<<(unsigned)((vecs + 255) / 256), 256, 0, stream>>>(static_cast<const uint4*>(dense_f16), vecs,
                                                                     static_cast<uint4*>(masked_f16),
                                                                     static_cast<uint2*>(mask_u8));
  return cudaGetLastError();
}

}  // namespace ob
