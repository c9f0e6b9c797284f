// K4: reference operand orders -> tile order, and tile order -> dense (the inverse of the pack).
//
// The reference hands its kernel a sign bitfield that is column-major in m and a metadata matrix in
// one of two shuffled orders (csrc/kernel.h:13-18, csrc/threadblock.h:198-199,
// onebit_sparse_mul/_semi_structured_conversions.py:21-48). The GEMM kernels of this library read
// 128x128 tiles whose sign bits are row-major in k and whose metadata is laid out for tensor
// memory. This kernel is the bit transpose between the two; one CTA per four vertically adjacent tiles, HBM-bound
// (3/16 byte read and written per dense weight). The operands must be 16-byte aligned.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "formats.h"
#include "kernels.h"

namespace {

// One CTA per column of kRB vertically adjacent 128 x 128 tiles. Everything enters and leaves the SM as 16-byte
// accesses: in the reference orders the sign bits of such a column are 64 segments of 16 * kRB bytes (128 * kRB rows of
// one bitfield column each) and its metadata is 4 runs of 512 * kRB bytes (one per pair of 16-column chunks: the row
// shuffles of both dialects stay inside a 128-row block). With kRB = 4 a segment is two whole 32-byte sectors and a
// CTA has 12 KiB of loads in flight; everything is requested before anything is used, staged in shared memory,
// permuted there, and stored in tile order (3 KiB contiguous per tile).
constexpr int kRB = 4;                                    // measured: 2 and 8 are slower at every size

// 32 x 32 bit transpose across a warp: lane l holds row l; afterwards bit l of lane j's word is what bit j of lane
// l's word was. Five butterfly stages of one shuffle each (a ballot per output word costs three times as much).
__device__ __forceinline__ uint32_t transpose32(uint32_t x, int lane) {
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) {
    const uint32_t m = s == 16 ? 0x0000ffffu : s == 8 ? 0x00ff00ffu : s == 4 ? 0x0f0f0f0fu : s == 2 ? 0x33333333u : 0x55555555u;
    const uint32_t y = __shfl_xor_sync(0xffffffffu, x, s);
    x = (lane & s) ? (((y >> s) & m) | (x & ~m)) : ((x & m) | ((y & m) << s));
  }
  return x;
}

__global__ void __launch_bounds__(256) ob_relayout_kernel(const uint8_t* __restrict__ bits_ref,
                                                          const uint16_t* __restrict__ meta_ref, int dialect,
                                                          int64_t m, int64_t k, uint32_t* __restrict__ bits_tile,
                                                          uint16_t* __restrict__ meta_tile) {
  __shared__ __align__(16) uint32_t s_bits[64 * kRB * 4];  // [kept value of the tile row][row block][32-row group]
  __shared__ __align__(16) uint16_t s_meta[4 * kRB * 256]; // [chunk pair][row block][shuffled row][2]
  __shared__ __align__(16) uint32_t s_out[kRB * 256];      // [row block] the tile's sign block in tile order
  const int64_t kb = blockIdx.x, mb0 = (int64_t)blockIdx.y * kRB;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int nrb = (int)min((int64_t)kRB, m / 128 - mb0);   // row blocks of this column that exist

  {
    constexpr int kBitPieces = 64 * kRB, kMetaPieces = 4 * kRB * 32;           // 16-byte pieces of the column
    constexpr int kBitLoads = (kBitPieces + 255) / 256, kMetaLoads = (kMetaPieces + 255) / 256;
    uint4 vb[kBitLoads], vm[kMetaLoads];
#pragma unroll
    for (int i = 0; i < kBitLoads; ++i) {
      const int idx = t + 256 * i, q = idx / kRB, rb = idx % kRB;                 // 64 segments x kRB pieces
      vb[i] = make_uint4(0, 0, 0, 0);
      if (idx < kBitPieces && rb < nrb) vb[i] = __ldg(reinterpret_cast<const uint4*>(bits_ref + ((kb * 64 + q) * m + (mb0 + rb) * 128) / 8));
    }
#pragma unroll
    for (int i = 0; i < kMetaLoads; ++i) {
      const int idx = t + 256 * i, pair = idx / (kRB * 32), rem = idx % (kRB * 32);   // 4 runs x kRB * 32 pieces
      vm[i] = make_uint4(0, 0, 0, 0);
      if (idx < kMetaPieces && rem / 32 < nrb) vm[i] = __ldg(reinterpret_cast<const uint4*>(meta_ref + (kb * 4 + pair) * 2 * m + mb0 * 256 + rem * 8));
    }
#pragma unroll
    for (int i = 0; i < kBitLoads; ++i)
      if (t + 256 * i < kBitPieces) reinterpret_cast<uint4*>(s_bits)[t + 256 * i] = vb[i];
#pragma unroll
    for (int i = 0; i < kMetaLoads; ++i)
      if (t + 256 * i < kMetaPieces) reinterpret_cast<uint4*>(s_meta)[t + 256 * i] = vm[i];
  }
  __syncthreads();

  // sign bits: warp = (32-row group, half of the 64 kept values). Lane l takes the bitfield word of the kept
  // value whose tile-order bit position is l; after the transpose lane j holds tile row j's word.
  {
    const int rg = warp & 3, half = warp >> 2;
    const int q_local = half * 32 + 2 * (lane & 15) + (lane >> 4);
    for (int rb = 0; rb < nrb; ++rb)
      s_out[rb * 256 + (rg * 32 + lane) * 2 + half] = transpose32(s_bits[(q_local * kRB + rb) * 4 + rg], lane);
  }
  // metadata: thread u < 128 of each half of the CTA assembles lane u of a tile block (8 words: chunk pairs
  // c2 = 0..3, rows r and r + 8); the two halves work on two row blocks at a time. Where a word comes from does
  // not depend on the row block.
  {
    const unsigned u = t & 127, r0 = u & 7, c1 = (u >> 3) & 1, r2 = u >> 4;
    unsigned src[8];
#pragma unroll
    for (unsigned wd = 0; wd < 8; ++wd) {
      const unsigned c2 = wd >> 1, r1 = wd & 1;
      unsigned rs, cs;
      ob_meta_ref_position_local(dialect, r0 + 8 * r1 + 16 * r2, 2 * c2 + c1, &rs, &cs);
      src[wd] = (cs >> 1) * (kRB * 256) + rs * 2 + (cs & 1);
    }
    for (int rb = t >> 7; rb < nrb; rb += 2) {
      __align__(16) uint16_t out[8];
#pragma unroll
      for (int wd = 0; wd < 8; ++wd) out[wd] = s_meta[src[wd] + rb * 256];
      reinterpret_cast<uint4*>(meta_tile)[((mb0 + rb) * (k / 128) + kb) * 128 + u] = *reinterpret_cast<const uint4*>(out);
    }
  }
  __syncthreads();
  for (int idx = t; idx < 64 * kRB; idx += 256) {
    const int rb = idx >> 6, i = idx & 63;
    if (rb < nrb) reinterpret_cast<uint4*>(bits_tile)[((mb0 + rb) * (k / 128) + kb) * 64 + i] = reinterpret_cast<const uint4*>(s_out)[idx];
  }
}

// tile order -> dense {-1, 0, +1} * scale, fp16 row-major (m, k). Used by the Python-level
// inverse (sparse_semi_structured_to_dense_cutlass / dequant_desparse_tile of the reference,
// _semi_structured_conversions.py:186-283, __init__.py:47-65) and by tests.
__global__ void __launch_bounds__(256) ob_tile_to_dense_kernel(const uint32_t* __restrict__ bits_tile,
                                                               const uint16_t* __restrict__ meta_tile,
                                                               const __half* __restrict__ scale, int64_t m, int64_t k,
                                                               __half* __restrict__ dense) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one (row, chunk) each
  const int64_t nchunks = k / 16;
  if (idx >= m * nchunks) return;
  const int64_t row = idx / nchunks, chunk = idx % nchunks;
  const unsigned meta = meta_tile[ob_meta_tile_offset(k, row, chunk)];
  const float s = scale ? __half2float(scale[row]) : 1.f;
  __align__(16) __half out[16];
#pragma unroll
  for (int t = 0; t < 16; ++t) out[t] = __float2half(0.f);
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    const int e = (meta >> (2 * t)) & 3;
    const int64_t bi = ob_bits_tile_index(k, row, chunk * 8 + t);
    const bool plus = (bits_tile[bi >> 5] >> (bi & 31)) & 1u;
    const __half v = __float2half(plus ? s : -s);
    const int pos = (t >> 1) * 4 + e;
#pragma unroll
    for (int p = 0; p < 16; ++p) if (p == pos) out[p] = v;
  }
  uint4* dst = reinterpret_cast<uint4*>(dense + row * k + chunk * 16);
  dst[0] = reinterpret_cast<uint4*>(out)[0];
  dst[1] = reinterpret_cast<uint4*>(out)[1];
}

}  // namespace

namespace ob {

cudaError_t launch_relayout(const void* bits_ref, const void* meta_ref, int dialect, int64_t m, int64_t k,
                            void* bits_tile, void* meta_tile, cudaStream_t stream) {
  // 16-byte accesses throughout; the reference's kernel asks the same of its A and E operands (128-bit alignment,
  // csrc/kernel.h:19-21 of the reference)
  if ((reinterpret_cast<uintptr_t>(bits_ref) | reinterpret_cast<uintptr_t>(meta_ref) | reinterpret_cast<uintptr_t>(bits_tile) |
       reinterpret_cast<uintptr_t>(meta_tile)) & 15)
    return cudaErrorMisalignedAddress;
  dim3 grid((unsigned)(k / 128), (unsigned)((m / 128 + kRB - 1) / kRB));
  ob_relayout_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(bits_ref),
                                               static_cast<const uint16_t*>(meta_ref), dialect, m, k,
                                               static_cast<uint32_t*>(bits_tile), static_cast<uint16_t*>(meta_tile));
  return cudaGetLastError();
}

cudaError_t launch_tile_to_dense(const void* bits_tile, const void* meta_tile, const void* scale, int64_t m,
                                 int64_t k, void* dense, cudaStream_t stream) {
  const int64_t items = m * (k / 16);
  ob_tile_to_dense_kernel<<<(unsigned)((items + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint32_t*>(bits_tile), static_cast<const uint16_t*>(meta_tile),
      static_cast<const __half*>(scale), m, k, static_cast<__half*>(dense));
  return cudaGetLastError();
}

}  // namespace ob
