// K3: the decode-regime kernel (few tokens, n <= 16 per pass): streams the 1.5 bit/weight operand
// from HBM exactly once and is meant to be bound by that stream, not by arithmetic.
//
// Replaces the reference's 128x64x128 CUTLASS threadblock (csrc/kernel.h:23-25) for the shapes
// where its 64-wide token tile is almost empty. Design:
//   * one CTA = one 128-row block of A x one slice of K; 8 warps, warp w owns rows 16w..16w+15;
//   * the K slices of one row block form a thread-block cluster (split-K). Partial sums are
//     reduced through distributed shared memory in a fixed order: deterministic, no atomics, no
//     scratch memory in HBM;
//   * every warp issues the loads of all its tiles of a chunk up front (16 B metadata + 16 B sign
//     words per lane and tile) so that a whole matrix of a few MiB is in flight at once;
//   * the 2:4 gather is done by the tensor core: sign words are expanded in registers to fp16 +-1
//     pairs (one shift + one logic op per pair, see the tile order in formats.h) and fed with the
//     metadata words to mma.sp m16n8k32 with fp32 accumulation;
//   * tokens (B, k x n row-major) are staged transposed in shared memory, zero-padded to 8 or 16.
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "formats.h"
#include "kernels.h"

namespace cg = cooperative_groups;

namespace {

constexpr int kChunkTiles = 4;                       // tiles (128 k each) whose loads are in flight together
constexpr int kChunkK = kChunkTiles * OB_TILE_K;     // 512
constexpr int kBtStride = kChunkK + 8;               // halves; +8 skews rows over the banks

__device__ __forceinline__ uint32_t expand_pair(uint32_t w, int j) {
  // bits j and 16+j of w -> fp16x2 {bit ? +1 : -1}
  return ((w << (15 - j)) & 0x80008000u) ^ 0xBC00BC00u;
}

__device__ __forceinline__ void mma_sp_16832(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[4],
                                             uint32_t e) {
  asm volatile(
      "mma.sp::ordered_metadata.sync.aligned.m16n8k32.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, "
      "{%4,%5,%6,%7}, {%8,%9,%10,%11}, {%0,%1,%2,%3}, %12, 0x0;\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(e));
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_stream8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

struct DecodeArgs {
  const uint8_t* bits_tile;
  const uint8_t* meta_tile;
  const __half* scale;
  const __half* b;
  void* d;
  int64_t m, n, k;
};

// NT = number of 8-token tiles per pass (1 or 2)
template <int NT, typename OutT>
__global__ void __launch_bounds__(256) ob_gemm_decode_kernel(DecodeArgs a) {
  constexpr int NP = NT * 8;
  __shared__ __align__(16) __half s_bt[NP * kBtStride];
  __shared__ __align__(16) float s_part[128 * NP];

  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int64_t mb = blockIdx.x;
  const int64_t n0 = (int64_t)blockIdx.z * NP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  const int64_t tiles_k = a.k / OB_TILE_K;
  const int64_t tile_begin = tiles_k * rank / S, tile_end = tiles_k * (rank + 1) / S;

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;

  const int u = g + 8 * (t & 1) + 16 * warp;                 // metadata lane of this thread
  const int row_lo = 16 * warp + g;

  for (int64_t chunk = tile_begin; chunk < tile_end; chunk += kChunkTiles) {
    const int ntile = (int)min((int64_t)kChunkTiles, tile_end - chunk);

    // 1. all weight loads of the chunk
    uint4 meta[kChunkTiles];
    uint2 blo[kChunkTiles], bhi[kChunkTiles];
#pragma unroll
    for (int ti = 0; ti < kChunkTiles; ++ti) {
      if (ti < ntile) {
        const int64_t tile = mb * tiles_k + chunk + ti;
        meta[ti] = ld_stream16(a.meta_tile + tile * OB_TILE_META_BYTES + u * 16);
        blo[ti] = ld_stream8(a.bits_tile + tile * OB_TILE_BITS_BYTES + row_lo * 8);
        bhi[ti] = ld_stream8(a.bits_tile + tile * OB_TILE_BITS_BYTES + (row_lo + 8) * 8);
      }
    }

    // 2. tokens of the chunk, transposed: s_bt[j][kk] = B[k0 + kk][n0 + j]
    const int64_t k0 = chunk * OB_TILE_K;
    const int kc = ntile * OB_TILE_K;
    __syncthreads();                                          // previous chunk's readers are done
    for (int idx = threadIdx.x; idx < kc * NP; idx += 256) {
      const int kk = idx / NP, j = idx % NP;
      const __half v = (n0 + j < a.n) ? a.b[(k0 + kk) * a.n + n0 + j] : __float2half(0.f);
      s_bt[j * kBtStride + kk] = v;
    }
    __syncthreads();

    // 3. four mma.sp per tile and token tile
#pragma unroll
    for (int ti = 0; ti < kChunkTiles; ++ti) {
      if (ti < ntile) {
        const uint32_t mw[4] = {meta[ti].x, meta[ti].y, meta[ti].z, meta[ti].w};
        const uint32_t wl[2] = {blo[ti].x, blo[ti].y}, wh[2] = {bhi[ti].x, bhi[ti].y};
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          const int j1 = 8 * (kb & 1) + t, j2 = j1 + 4;
          uint32_t af[4];
          af[0] = expand_pair(wl[kb >> 1], j1);
          af[1] = expand_pair(wh[kb >> 1], j1);
          af[2] = expand_pair(wl[kb >> 1], j2);
          af[3] = expand_pair(wh[kb >> 1], j2);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint32_t* brow = reinterpret_cast<const uint32_t*>(s_bt + (nt * 8 + g) * kBtStride + ti * OB_TILE_K + kb * 32);
            uint32_t bf[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) bf[i] = brow[t + 4 * i];
            mma_sp_16832(acc[nt], af, bf, mw[kb]);
          }
        }
      }
    }
  }

  // split-K reduction through distributed shared memory, fixed order
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    s_part[row_lo * NP + nt * 8 + 2 * t] = acc[nt][0];
    s_part[row_lo * NP + nt * 8 + 2 * t + 1] = acc[nt][1];
    s_part[(row_lo + 8) * NP + nt * 8 + 2 * t] = acc[nt][2];
    s_part[(row_lo + 8) * NP + nt * 8 + 2 * t + 1] = acc[nt][3];
  }
  cluster.sync();
  const int rows_per = 128 / S;
  for (int e = threadIdx.x; e < rows_per * NP; e += 256) {
    const int r = rank * rows_per + e / NP, j = e % NP;
    float sum = 0.f;
    for (int s = 0; s < S; ++s) sum += cluster.map_shared_rank(s_part, s)[r * NP + j];
    const int64_t row = mb * 128 + r;
    if (a.scale) sum *= __half2float(a.scale[row]);
    if (n0 + j < a.n) {
      if constexpr (sizeof(OutT) == 2) static_cast<__half*>(a.d)[row * a.n + n0 + j] = __float2half_rn(sum);
      else static_cast<float*>(a.d)[row * a.n + n0 + j] = sum;
    }
  }
  cluster.sync();                                             // keep s_part alive until every peer has read it
}

template <int NT, typename OutT>
cudaError_t launch(const DecodeArgs& a, int S, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(a.m / 128), (unsigned)S, (unsigned)((a.n + NT * 8 - 1) / (NT * 8)));
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)S;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, ob_gemm_decode_kernel<NT, OutT>, a);
}

}  // namespace

namespace ob {

cudaError_t launch_gemm_decode(const void* bits_tile, const void* meta_tile, const void* scale, const void* b,
                               void* d, int64_t m, int64_t n, int64_t k, int out_type, cudaStream_t stream) {
  DecodeArgs a{static_cast<const uint8_t*>(bits_tile), static_cast<const uint8_t*>(meta_tile),
               static_cast<const __half*>(scale), static_cast<const __half*>(b), d, m, n, k};
  // split K over a cluster of up to 8 CTAs, as far as there are tiles and until the grid holds
  // about four CTAs per SM
  const int64_t tiles_k = k / OB_TILE_K, row_blocks = m / 128;
  int S = 1;
  while (S < 8 && 2 * S <= tiles_k && row_blocks * S < 4 * 148) S *= 2;
  const bool two = (n > 8);
  if (out_type == OB_OUT_F16) return two ? launch<2, __half>(a, S, stream) : launch<1, __half>(a, S, stream);
  return two ? launch<2, float>(a, S, stream) : launch<1, float>(a, S, stream);
}

}  // namespace ob
