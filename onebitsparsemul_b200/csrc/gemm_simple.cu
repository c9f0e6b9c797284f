// Plain CUDA-core kernel on the reference operand orders: one thread per output element, fp32
// accumulation in increasing k, exactly the arithmetic of the reference's host check
// (tests/kernel_test.cu:441-456 with the bit -> +-1 rule of csrc/warp.h:40-51). It exists to state
// every layout fact of the reference in the simplest possible device code, to serve shapes the
// tiled kernels do not take (m or k not a multiple of 128), and as an on-device cross-check.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "formats.h"
#include "kernels.h"

namespace {

template <typename OutT>
__global__ void __launch_bounds__(256) ob_gemm_simple_kernel(const uint8_t* __restrict__ bits_ref,
                                                             const uint16_t* __restrict__ meta_ref, int dialect,
                                                             const __half* __restrict__ scale,
                                                             const __half* __restrict__ b, OutT* __restrict__ d,
                                                             int64_t m, int64_t n, int64_t k) {
  const int64_t j = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;   // n fastest: coalesced B and D
  const int64_t i = blockIdx.x;
  if (j >= n) return;
  float acc = 0.f;
  for (int64_t c = 0; c < k / 16; ++c) {
    const unsigned w = meta_ref[ob_meta_ref_offset(dialect, m, i, c)];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int e = (w >> (2 * t)) & 3;
      const int64_t idx = ob_bits_ref_index(m, i, c * 8 + t);
      const bool plus = (bits_ref[idx >> 3] >> (idx & 7)) & 1u;
      const float v = __half2float(b[(c * 16 + (t >> 1) * 4 + e) * n + j]);
      acc += plus ? v : -v;
    }
  }
  if (scale) acc *= __half2float(scale[i]);
  if constexpr (sizeof(OutT) == 2) d[i * n + j] = __float2half_rn(acc);
  else d[i * n + j] = acc;
}

}  // namespace

namespace ob {

cudaError_t launch_gemm_simple(const void* bits_ref, const void* meta_ref, int dialect, const void* scale,
                               const void* b, void* d, int64_t m, int64_t n, int64_t k, int out_type,
                               cudaStream_t stream) {
  dim3 grid((unsigned)m, (unsigned)((n + 255) / 256));
  if (out_type == OB_OUT_F16)
    ob_gemm_simple_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(bits_ref),
        static_cast<const uint16_t*>(meta_ref), dialect, static_cast<const __half*>(scale),
        static_cast<const __half*>(b), static_cast<__half*>(d), m, n, k);
  else
    ob_gemm_simple_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(bits_ref),
        static_cast<const uint16_t*>(meta_ref), dialect, static_cast<const __half*>(scale),
        static_cast<const __half*>(b), static_cast<float*>(d), m, n, k);
  return cudaGetLastError();
}

}  // namespace ob
