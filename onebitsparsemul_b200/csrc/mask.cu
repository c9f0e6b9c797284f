// Magnitude 2:4 mask: in every group of 4 consecutive weights drop the two smallest |w|.
// Replaces mask_creator (onebit_sparse_mul/_semi_structured_conversions.py:286-314: abs, argsort per
// group of 4, scatter zeros), the slowest step of the reference's pack(). torch.argsort leaves the
// order of equal magnitudes unspecified; here the lower index is dropped first. One thread per 8
// weights (two groups, one 16-byte load); HBM-bound.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "pack16.h"

namespace {

__global__ void __launch_bounds__(256) ob_mask24_kernel(const uint4* __restrict__ dense, int64_t vecs,
                                                        uint4* __restrict__ masked, uint2* __restrict__ mask) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= vecs) return;
  uint4 v = __ldg(dense + i);
  uint32_t k0, k1, k2, k3;                                  // bit 15 / 31: the weight in that half stays
  ob_keep_group2(v.x, v.y, k0, k1);
  ob_keep_group2(v.z, v.w, k2, k3);
  if (mask) {
    // one byte per weight, 1 = kept: bit 15 -> bit 0 of byte 0, bit 31 -> bit 0 of byte 1 of each pair
    const uint32_t b0 = (k0 >> 15) & 1u, b1 = (k0 >> 23) & 0x100u, b2 = (k1 >> 15) & 1u, b3 = (k1 >> 23) & 0x100u;
    const uint32_t b4 = (k2 >> 15) & 1u, b5 = (k2 >> 23) & 0x100u, b6 = (k3 >> 15) & 1u, b7 = (k3 >> 23) & 0x100u;
    mask[i] = make_uint2(b0 | b1 | ((b2 | b3) << 16), b4 | b5 | ((b6 | b7) << 16));
  }
  if (masked) {
    // the reference multiplies by the 0/1 mask: a dropped weight becomes a signed zero, a NaN stays a NaN
    const uint32_t p0 = k0 | ob_nan2(v.x, 0x03ff03ffu), p1 = k1 | ob_nan2(v.y, 0x03ff03ffu);
    const uint32_t p2 = k2 | ob_nan2(v.z, 0x03ff03ffu), p3 = k3 | ob_nan2(v.w, 0x03ff03ffu);
    v.x &= ((p0 >> 15) * 0xffffu) | kObSign2;
    v.y &= ((p1 >> 15) * 0xffffu) | kObSign2;
    v.z &= ((p2 >> 15) * 0xffffu) | kObSign2;
    v.w &= ((p3 >> 15) * 0xffffu) | kObSign2;
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
