// K1: 2:4 compress + metadata encode + one-bit quantise + bit-pack, one pass over the dense matrix.
//
// Replaces the torch-op chain of the reference's BinaryLinear_2_4.pack
// (onebit_sparse_mul/__init__.py:130-145): sparse_semi_structured_from_dense_cutlass
// (_semi_structured_conversions.py:54-179) -> binary_quant (__init__.py:22-23) -> .T ->
// pack_binary (__init__.py:25-34). All outputs are bit-exact with that chain.
//
// One CTA owns one 128-row x 128-column tile. A warp owns 32 rows of one 16-column chunk, lane =
// row, so that the column-major-in-m sign bitfield of the reference falls out of warp ballots and
// the 4 nibbles of a chunk are one lane's private work. 16-bit weights enter the SM as coalesced 16-byte
// loads (a quarter-warp reads 128 contiguous bytes of a row) into a padded shared-memory tile, from which a
// lane then takes its 32 bytes without bank conflicts; everything leaves the SM as 16-byte stores.
// HBM-bound: 2 bytes read and at most ~0.6 byte written per dense weight.
//
// Fused form (fp16 only): the 2:4 magnitude mask of mask_creator (_semi_structured_conversions.py:286-314)
// is applied to the 16 values a lane has just loaded, before they are encoded, so that the whole of
// BinaryLinear_2_4.pack -- mask, compress, encode, quantise, bit-pack -- is ONE pass over the dense weights:
// the masked copy is never written and read back (it is written only if the caller asks for it).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "formats.h"
#include "kernels.h"
#include "pack16.h"

namespace {

// The per-weight tests of a chunk as half2 comparisons: one FMA-pipe instruction per register of two weights and
// test, where the integer forms of pack16.h take three to four ALU-pipe instructions (the kernel is bound by the
// ALU pipe). A comparison mask is 0xffff in the halves where it holds.
//   non-zero = unordered-or-not-equal to 0 (a NaN is non-zero, -0 is not)
//   positive = greater than 0 (false for a NaN, for +-0 and for negative values; true for +inf and subnormals)
template <int DT> __device__ __forceinline__ void chunk_masks(const uint32_t (&x)[8], uint32_t& M, uint32_t& P) {
  uint32_t m2 = 0, p2 = 0;                                 // bits 2i and 16 + 2i: weights 2i and 2i + 1
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t nz, pos;
    if constexpr (DT == OB_DENSE_F16) {
      const __half2 v = *reinterpret_cast<const __half2*>(&x[i]), z = __half2half2(__ushort_as_half(0));
      nz = __hneu2_mask(v, z);
      pos = __hgt2_mask(v, z);
    } else {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&x[i]), z = __bfloat162bfloat162(__ushort_as_bfloat16(0));
      nz = __hneu2_mask(v, z);
      pos = __hgt2_mask(v, z);
    }
    m2 |= nz & (0x00010001u << (2 * i));
    p2 |= pos & (0x00010001u << (2 * i));
  }
  M = (m2 | (m2 >> 15)) & 0xffffu;
  P = (p2 | (p2 >> 15)) & 0xffffu;
}

// ob_mask_group2 of pack16.h with the NaN test as a half2 comparison (x != x)
__device__ __forceinline__ void mask_group2_f16(uint32_t& w0, uint32_t& w1) {
  uint32_t keep0, keep1;
  ob_keep_group2(w0, w1, keep0, keep1);
  const __half2 h0 = *reinterpret_cast<const __half2*>(&w0), h1 = *reinterpret_cast<const __half2*>(&w1);
  w0 &= ((keep0 >> 15) * 0xffffu) | __hneu2_mask(h0, h0) | kObSign2;
  w1 &= ((keep1 >> 15) * 0xffffu) | __hneu2_mask(h1, h1) | kObSign2;
}

template <int DT> struct DenseTraits;
template <> struct DenseTraits<OB_DENSE_F16> {
  using T = uint16_t;
  __device__ static bool nonzero(T v) { return (v & 0x7fffu) != 0; }
  __device__ static bool positive(T v) { const unsigned mag = v & 0x7fffu; return !(v & 0x8000u) && mag != 0 && mag <= 0x7c00u; }
};
template <> struct DenseTraits<OB_DENSE_BF16> {
  using T = uint16_t;
  __device__ static bool nonzero(T v) { return (v & 0x7fffu) != 0; }
  __device__ static bool positive(T v) { const unsigned mag = v & 0x7fffu; return !(v & 0x8000u) && mag != 0 && mag <= 0x7f80u; }
};
template <> struct DenseTraits<OB_DENSE_I32> {
  using T = int32_t;
  __device__ static bool nonzero(T v) { return v != 0; }
  __device__ static bool positive(T v) { return v > 0; }
};

struct PackArgs {
  const void* dense;
  int64_t m, k;
  void* sparse;        // (m, k/2) kept values, dense dtype            (nullable)
  uint8_t* bits_ref;   // (k/2, m/8) reference A bitfield              (nullable)
  uint16_t* meta_ref;  // (m, k/16) reference-ordered metadata         (nullable)
  int dialect;
  uint32_t* bits_tile; // tile-ordered sign bits                       (nullable; needs m,k % 128 == 0)
  uint16_t* meta_tile; // tile-ordered metadata                        (nullable; needs m,k % 128 == 0)
  int apply_mask;      // fp16 only: mask every group of 4 to its two largest magnitudes first
  void* masked;        // (m, k) the masked weights, fp16                (nullable; with apply_mask)
};

template <int DT>
__global__ void __launch_bounds__(256) ob_pack_kernel(PackArgs a) {
  using Tr = DenseTraits<DT>;
  using T = typename Tr::T;
  constexpr int kElemsPer16B = 16 / sizeof(T);

  __shared__ __align__(16) uint16_t s_meta_tile[1024];     // 2 KiB, tile order
  __shared__ __align__(16) uint32_t s_bits_tile[256];      // 1 KiB, tile order
  __shared__ __align__(16) uint32_t s_bits_ref[64 * 4];    // [q local][32-row group]
  __shared__ __align__(16) uint16_t s_meta_ref[4 * 256];   // [chunk pair][shuffled row][2]

  // 16-bit weights: the dense tile itself, rows 272 bytes apart (lanes of a quarter-warp, one row each, then hit
  // disjoint banks with their 16-byte accesses)
  constexpr bool kStaged = sizeof(T) == 2;
  constexpr int kRowStride = 136;                            // uint16 per staged row
  __shared__ __align__(16) uint16_t s_dense[kStaged ? 128 * kRowStride : 8];

  const int64_t kb = blockIdx.x, mb = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nchunks = a.k / 16;

  if constexpr (kStaged) {
    uint4 stage[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = threadIdx.x + 256 * i, r = idx >> 4, c8 = idx & 15;   // row of the tile, 8-value piece of the row
      const int64_t row = mb * 128 + r, col = kb * 128 + c8 * 8;
      stage[i] = (row < a.m && col < a.k) ? __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.dense) + row * a.k + col))
                                          : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = threadIdx.x + 256 * i, r = idx >> 4, c8 = idx & 15;
      *reinterpret_cast<uint4*>(&s_dense[r * kRowStride + c8 * 8]) = stage[i];
    }
  }
  s_bits_tile[threadIdx.x] = 0;
  s_bits_ref[threadIdx.x] = 0;
  for (int i = threadIdx.x; i < 1024; i += 256) { s_meta_tile[i] = 0; s_meta_ref[i] = 0; }
  __syncthreads();

  for (int item = warp; item < 32; item += 8) {
    const int rg = item & 3, c = item >> 2;             // 32-row group, chunk inside the tile
    const int r = rg * 32 + lane;                       // row inside the tile
    const int64_t row = mb * 128 + r, chunk = kb * 8 + c;
    const bool valid = row < a.m && chunk < nchunks;

    unsigned meta = 0, even = 0, odd = 0;               // metadata word; signs of the first / second kept weight of each group
    if constexpr (kStaged) {
      // 16-bit weights, two per register: mask, tests and encoder work on both halves and on all four groups at once
      // (pack16.h). Rows and columns beyond the matrix were staged as zeros.
      uint32_t x[8];
      *reinterpret_cast<uint4*>(&x[0]) = *reinterpret_cast<const uint4*>(&s_dense[r * kRowStride + c * 16]);
      *reinterpret_cast<uint4*>(&x[4]) = *reinterpret_cast<const uint4*>(&s_dense[r * kRowStride + c * 16 + 8]);
      if constexpr (DT == OB_DENSE_F16) {
        if (a.apply_mask) {
#pragma unroll
          for (int g = 0; g < 4; ++g) mask_group2_f16(x[2 * g], x[2 * g + 1]);
          if (a.masked) {                                 // back into the staged tile; stored row-wise at the end
            *reinterpret_cast<uint4*>(&s_dense[r * kRowStride + c * 16]) = *reinterpret_cast<uint4*>(&x[0]);
            *reinterpret_cast<uint4*>(&s_dense[r * kRowStride + c * 16 + 8]) = *reinterpret_cast<uint4*>(&x[4]);
          }
        }
      }
      uint32_t M, P, s0, s1;
      chunk_masks<DT>(x, M, P);
      meta = ob_encode_planes(M, P, s0, s1);
      // reference bitfield: one ballot per kept value gives 32 rows of one bitfield column
      if (a.bits_ref) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const unsigned w = __ballot_sync(0xffffffffu, valid && ((((t & 1) ? s1 : s0) >> (4 * (t >> 1))) & 1u));
          if (lane == 0) s_bits_ref[(c * 8 + t) * 4 + rg] = w;
        }
      }
      if (!valid) continue;
      even = ob_plane_to_nibble(s0);
      odd = ob_plane_to_nibble(s1);
      if (a.sparse) {                                     // the kept values themselves (exchange format, tests)
        const T* e = reinterpret_cast<const T*>(x);
        T kept[8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int i0 = (meta >> (4 * g)) & 3, i1 = (meta >> (4 * g + 2)) & 3;
          kept[2 * g] = i0 == 0 ? e[4 * g] : i0 == 1 ? e[4 * g + 1] : e[4 * g + 2];
          kept[2 * g + 1] = i1 == 1 ? e[4 * g + 1] : i1 == 2 ? e[4 * g + 2] : e[4 * g + 3];
        }
        *reinterpret_cast<uint4*>(static_cast<T*>(a.sparse) + row * (a.k / 2) + chunk * 8) = *reinterpret_cast<uint4*>(kept);
      }
    } else {
      T e[16];
      if (valid) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(a.dense) + row * a.k + chunk * 16);
#pragma unroll
        for (int v = 0; v < 16 / kElemsPer16B; ++v) {
          const uint4 x = __ldg(src + v);
          *reinterpret_cast<uint4*>(&e[v * kElemsPer16B]) = x;
        }
      } else {
#pragma unroll
        for (int t = 0; t < 16; ++t) e[t] = T(0);
      }
      unsigned signs = 0;
      T kept[8];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const unsigned nib = ob_encode_group(Tr::nonzero(e[4 * g]), Tr::nonzero(e[4 * g + 1]),
                                             Tr::nonzero(e[4 * g + 2]), Tr::nonzero(e[4 * g + 3]));
        meta |= nib << (4 * g);
        const int i0 = nib & 3, i1 = nib >> 2;
        // a 4-way select keeps e[] in registers (no dynamic indexing)
        const T v0 = i0 == 0 ? e[4 * g] : i0 == 1 ? e[4 * g + 1] : e[4 * g + 2];
        const T v1 = i1 == 1 ? e[4 * g + 1] : i1 == 2 ? e[4 * g + 2] : e[4 * g + 3];
        kept[2 * g] = v0; kept[2 * g + 1] = v1;
        signs |= (Tr::positive(v0) ? 1u : 0u) << (2 * g);
        signs |= (Tr::positive(v1) ? 1u : 0u) << (2 * g + 1);
      }
      // reference bitfield: one ballot per kept value gives 32 rows of one bitfield column
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const unsigned w = __ballot_sync(0xffffffffu, valid && ((signs >> t) & 1u));
        if (lane == 0) s_bits_ref[(c * 8 + t) * 4 + rg] = w;
      }
      if (!valid) continue;
      if (a.sparse) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(a.sparse) + row * (a.k / 2) + chunk * 8);
#pragma unroll
        for (int v = 0; v < 8 / kElemsPer16B; ++v) dst[v] = *reinterpret_cast<uint4*>(&kept[v * kElemsPer16B]);
      }
      even = (signs & 1u) | ((signs >> 1) & 2u) | ((signs >> 2) & 4u) | ((signs >> 3) & 8u);
      odd = ((signs >> 1) & 1u) | ((signs >> 2) & 2u) | ((signs >> 3) & 4u) | ((signs >> 4) & 8u);
    }
    // tile-ordered metadata
    {
      const int r0 = r & 7, r1 = (r >> 3) & 1, r2 = r >> 4, c1 = c & 1, c2 = c >> 1;
      s_meta_tile[(r0 + 8 * c1 + 16 * r2) * 8 + 2 * c2 + r1] = (uint16_t)meta;
    }
    // tile-ordered sign bits: even kept values to bits 4*(c&3).., odd ones 16 higher
    atomicOr(&s_bits_tile[r * 2 + (c >> 2)], (even << (4 * (c & 3))) | (odd << (16 + 4 * (c & 3))));
    // reference-ordered metadata: destination stays inside this tile's 4 chunk pairs x 128 rows
    if (a.meta_ref) {
      unsigned rs, cs;                                                  // shuffled row and column inside the tile
      ob_meta_ref_position_local(a.dialect, (unsigned)r, (unsigned)c, &rs, &cs);
      s_meta_ref[(cs >> 1) * 256 + rs * 2 + (cs & 1)] = (uint16_t)meta;
    }
  }
  __syncthreads();

  const int t = threadIdx.x;
  const bool full = (mb * 128 + 128 <= a.m) && (kb * 128 + 128 <= a.k);
  if constexpr (DT == OB_DENSE_F16) {
    if (a.apply_mask && a.masked) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = t + 256 * i, r = idx >> 4, c8 = idx & 15;
        const int64_t row = mb * 128 + r, col = kb * 128 + c8 * 8;
        if (row < a.m && col < a.k)
          *reinterpret_cast<uint4*>(static_cast<T*>(a.masked) + row * a.k + col) = *reinterpret_cast<const uint4*>(&s_dense[r * kRowStride + c8 * 8]);
      }
    }
  }
  if (a.meta_tile && full && t < 128)
    reinterpret_cast<uint4*>(a.meta_tile)[(mb * (a.k / 128) + kb) * 128 + t] = reinterpret_cast<uint4*>(s_meta_tile)[t];
  if (a.bits_tile && full && t >= 128 && t < 192)
    reinterpret_cast<uint4*>(a.bits_tile)[(mb * (a.k / 128) + kb) * 64 + (t - 128)] = reinterpret_cast<uint4*>(s_bits_tile)[t - 128];
  if (a.bits_ref) {
    // s_bits_ref row q = 16 bytes = rows 128*mb .. +127 of bitfield column q
    if (full) {
      if (t < 64)
        *reinterpret_cast<uint4*>(a.bits_ref + ((kb * 64 + t) * a.m + mb * 128) / 8) = reinterpret_cast<uint4*>(s_bits_ref)[t];
    } else {
      const uint8_t* sb = reinterpret_cast<const uint8_t*>(s_bits_ref);
      for (int i = t; i < 64 * 16; i += 256) {
        const int64_t q = kb * 64 + (i >> 4), rbyte = mb * 16 + (i & 15);
        if (q < a.k / 2 && rbyte < a.m / 8) a.bits_ref[q * (a.m / 8) + rbyte] = sb[i];
      }
    }
  }
  if (a.meta_ref) {
    if (full) {
      if (t < 128) {
        const int pair = t >> 5, j = t & 31;        // 512 B per pair = 32 x 16 B
        *reinterpret_cast<uint4*>(a.meta_ref + (kb * 4 + pair) * 2 * a.m + mb * 256 + j * 8) =
            reinterpret_cast<uint4*>(s_meta_ref)[t];
      }
    } else {
      for (int i = t; i < 1024; i += 256) {
        const int64_t pair = kb * 4 + (i >> 8), rest = mb * 256 + (i & 255);
        // a chunk pair exists if its first chunk does; an odd chunk count never happens with a
        // second chunk missing inside a pair because the 2x2 swap needs both columns
        if (pair * 2 < nchunks && rest < 2 * a.m && (pair * 2 + 1 < nchunks || (rest & 1) == 0))
          a.meta_ref[pair * 2 * a.m + rest] = s_meta_ref[i];
      }
    }
  }
}

}  // namespace

namespace ob {

cudaError_t launch_pack(const void* dense, int dense_dtype, int64_t m, int64_t k, void* sparse,
                        void* bits_ref, void* meta_ref, int dialect, void* bits_tile, void* meta_tile,
                        bool apply_mask, void* masked, cudaStream_t stream) {
  if (apply_mask && dense_dtype != OB_DENSE_F16) return cudaErrorInvalidValue;
  PackArgs a{dense, m, k, sparse, static_cast<uint8_t*>(bits_ref), static_cast<uint16_t*>(meta_ref),
             dialect, static_cast<uint32_t*>(bits_tile), static_cast<uint16_t*>(meta_tile), apply_mask ? 1 : 0, masked};
  dim3 grid((unsigned)((k + 127) / 128), (unsigned)((m + 127) / 128));
  switch (dense_dtype) {
    case OB_DENSE_F16: ob_pack_kernel<OB_DENSE_F16><<<grid, 256, 0, stream>>>(a); break;
    case OB_DENSE_BF16: ob_pack_kernel<OB_DENSE_BF16><<<grid, 256, 0, stream>>>(a); break;
    case OB_DENSE_I32: ob_pack_kernel<OB_DENSE_I32><<<grid, 256, 0, stream>>>(a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace ob
