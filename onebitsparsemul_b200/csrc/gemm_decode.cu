// K3: the decode-regime kernel (few tokens, n <= 16 per pass): streams the 1.5 bit/weight operand
// from HBM exactly once and is meant to be bound by that stream, not by arithmetic.
//
// Replaces the reference's 128x64x128 CUTLASS threadblock (csrc/kernel.h:23-25) for the shapes
// where its 64-wide token tile is almost empty. Such a call moves only a few MiB, so the kernel is
// built to be short: every weight load of a warp is issued before anything else, and there is one
// cluster-wide synchronisation in its whole life.
//   * one CTA = one 128-row block of A x one slice of K, 16 warps: warp w owns rows 16(w%8)..+15 of
//     half (w/8) of the slice, so a cluster of S CTAs cuts K into 2S slices;
//   * the 2:4 gather is done by the tensor core: sign words are expanded in registers to fp16 +-1
//     pairs (one shift + one logic op per pair, see the tile order in formats.h) and fed with the
//     metadata words to mma.sp m16n8k32 with fp32 accumulation;
//   * tokens (B, k x n row-major) are staged TRANSPOSED in shared memory (one padded row per token,
//     zero rows beyond n) by the half that uses them (named barrier per half), so that a B fragment
//     register is one 32-bit load;
//   * split-K reduction: every warp PUSHES its partial sums through distributed shared memory into
//     the CTA that owns those output rows; after the single cluster barrier each CTA sums its 2S
//     slices in a fixed order from its own shared memory, scales, converts and stores. No atomics,
//     no scratch in HBM, no remote reads, deterministic.
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "formats.h"
#include "kernels.h"

namespace cg = cooperative_groups;

namespace {

// Timeline instrumentation for tuning, compiled in only with -DOB_TRACE.
#ifdef OB_TRACE
__device__ long long g_trace_dec[4][16];
#define OB_TRACE_EV(ev) do { if (blockIdx.x == 3 && blockIdx.z == 0 && (threadIdx.x == 0 || threadIdx.x == 511) && blockIdx.y < 2) g_trace_dec[blockIdx.y * 2 + (threadIdx.x != 0)][ev] = clock64(); } while (0)
#else
#define OB_TRACE_EV(ev) do { } while (0)
#endif

constexpr int kChunkTiles = 3;                       // tiles (128 k each) of one warp in flight together
constexpr int kChunkK = kChunkTiles * OB_TILE_K;     // 384
constexpr int kMaxSlices = 16;                       // 2 halves x cluster of up to 8
constexpr int kBtStride = kChunkK + 8;               // halves per token column; +8 skews the columns over the banks

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
__device__ __forceinline__ void half_barrier(int half) {      // the 256 threads of one half of the CTA
  asm volatile("bar.sync %0, 256;" ::"r"(half + 1) : "memory");
}

struct DecodeArgs {
  const uint8_t* bits_tile;
  const uint8_t* meta_tile;
  const __half* scale;
  const __half* bias;   // per output row, added after the scale (token-major callers; NULL = none)
  const __half* b;
  void* d;
  int64_t m, n, k;
};

// NT = number of 8-token tiles per pass (1 or 2)
// TM = token-major operands (the nn.Linear convention): b is x (n, k) row-major, d is y (n, m) row-major
template <int NT, typename OutT, bool TM>
__global__ void __launch_bounds__(512, 2) ob_gemm_decode_kernel(DecodeArgs a) {
  constexpr int NP = NT * 8;
  __shared__ __align__(16) __half s_b[2][NP * kBtStride];          // per half: s_b[j][kk] = B[k0 + kk][n0 + j]
  __shared__ __align__(16) float s_recv[kMaxSlices * 16 * NP];    // [slice][row of this CTA's share][token]

  OB_TRACE_EV(0);
  // the cluster spans the whole y extent of the grid: rank and size come from the launch geometry,
  // which is cheaper to read at kernel start than the cluster special registers
  const int S = (int)gridDim.y;
  const int rank = (int)blockIdx.y;
  const int64_t mb = blockIdx.x;
  const int64_t n0 = (int64_t)blockIdx.z * NP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = warp >> 3, w8 = warp & 7;                  // K half, 16-row block
  const int tid_h = threadIdx.x & 255;                        // thread index inside the half
  const int g = lane >> 2, t = lane & 3;

  const int64_t tiles_k = a.k / OB_TILE_K;
  const int slices = 2 * S, slice = 2 * rank + half;
  const int64_t tile_begin = tiles_k * slice / slices, tile_end = tiles_k * (slice + 1) / slices;

  const int u = g + 8 * (t & 1) + 16 * w8;                    // metadata lane of this thread
  const int row_lo = 16 * w8 + g;

  // 1. the weight loads of the first chunk, before anything else
  uint4 meta[kChunkTiles];
  uint2 blo[kChunkTiles], bhi[kChunkTiles];
  auto load_chunk = [&](int64_t chunk) {
#pragma unroll
    for (int ti = 0; ti < kChunkTiles; ++ti) {
      if (chunk + ti < tile_end) {
        const int64_t tile = mb * tiles_k + chunk + ti;
        meta[ti] = ld_stream16(a.meta_tile + tile * OB_TILE_META_BYTES + u * 16);
        blo[ti] = ld_stream8(a.bits_tile + tile * OB_TILE_BITS_BYTES + row_lo * 8);
        bhi[ti] = ld_stream8(a.bits_tile + tile * OB_TILE_BITS_BYTES + (row_lo + 8) * 8);
      }
    }
  };
  load_chunk(tile_begin);
  OB_TRACE_EV(1);

  // two independent accumulation chains per token tile (even / odd k-blocks): the warp-level MMA has
  // a long latency and a single chain would serialise on it
  float acc[2][NT][4];
#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[c][nt][i] = 0.f;

  const int nvalid = (int)min((int64_t)NP, a.n - n0);
  const bool vec_rows = !TM && (a.n % 8 == 0) && (nvalid == NP) && ((reinterpret_cast<uintptr_t>(a.b) & 15) == 0);
  __half* sb = s_b[half];

  for (int64_t chunk = tile_begin; chunk < tile_end; chunk += kChunkTiles) {
    const int ntile = (int)min((int64_t)kChunkTiles, tile_end - chunk);
    if (chunk != tile_begin) {
      half_barrier(half);                                     // previous chunk's readers are done
      load_chunk(chunk);
    }
    // 2. tokens of the chunk: sb[kk][j] = B[k0 + kk][n0 + j], zero beyond n
    const int64_t k0 = chunk * OB_TILE_K;
    const int kc = ntile * OB_TILE_K;
    if constexpr (TM) {
      // token j is a contiguous row of x: 16-byte pieces along k, zero rows beyond n
      const int pieces = kc / 8;
      for (int idx = tid_h; idx < NP * pieces; idx += 256) {
        const int j = idx / pieces, pc = idx - j * pieces;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (j < nvalid) v = __ldg(reinterpret_cast<const uint4*>(a.b + (n0 + j) * a.k + k0 + pc * 8));
        *reinterpret_cast<uint4*>(&sb[j * kBtStride + pc * 8]) = v;
      }
    } else if (vec_rows) {
      constexpr int kPieces = NP / 8;                         // 16-byte pieces per token row
      for (int idx = tid_h; idx < kc * kPieces; idx += 256) {
        const int kk = idx / kPieces, pc = idx % kPieces;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.b + (k0 + kk) * a.n + n0 + pc * 8));
        const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) sb[(pc * 8 + jj) * kBtStride + kk] = h[jj];
      }
    } else {
      for (int kk = tid_h; kk < kc; kk += 256) {
#pragma unroll
        for (int j = 0; j < NP; ++j) sb[j * kBtStride + kk] = (j < nvalid) ? a.b[(k0 + kk) * a.n + n0 + j] : __float2half(0.f);
      }
    }
    OB_TRACE_EV(2);
    half_barrier(half);
    OB_TRACE_EV(3);

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
            // fragment register i: token column nt*8+g, k rows 2t+8i and 2t+8i+1 of the k-block
            const uint32_t* brow = reinterpret_cast<const uint32_t*>(sb + (nt * 8 + g) * kBtStride + ti * OB_TILE_K + kb * 32);
            uint32_t bf[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) bf[i] = brow[t + 4 * i];
            mma_sp_16832(acc[kb & 1][nt], af, bf, mw[kb]);
          }
        }
      }
    }
  }

  OB_TRACE_EV(4);
  // 4. push the partial sums to the CTA that owns the rows: CTA r owns rows [r * 128/S, (r+1) * 128/S)
  cg::cluster_group cluster = cg::this_cluster();
  const int rows_per = 128 / S;
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    const int r = row_lo + 8 * hrow;
    float* dst = cluster.map_shared_rank(s_recv, r / rows_per) + (slice * rows_per + (r % rows_per)) * NP;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      *reinterpret_cast<float2*>(dst + nt * 8 + 2 * t) = make_float2(acc[0][nt][2 * hrow] + acc[1][nt][2 * hrow],
                                                                   acc[0][nt][2 * hrow + 1] + acc[1][nt][2 * hrow + 1]);
  }
  OB_TRACE_EV(5);
  cluster.sync();                                             // the only cluster-wide barrier
  OB_TRACE_EV(6);

  // 5. fixed-order sum of the 2S slices from this CTA's own shared memory
  for (int e = threadIdx.x; e < rows_per * NP; e += 512) {
    // consecutive threads walk the fastest output dimension: tokens of a row (m x n), rows of a token (n x m)
    const int rr = TM ? e % rows_per : e / NP, j = TM ? e / rows_per : e % NP;
    float sum = 0.f;
    for (int sl = 0; sl < slices; ++sl) sum += s_recv[(sl * rows_per + rr) * NP + j];
    const int64_t row = mb * 128 + rank * rows_per + rr;
    if (a.scale) sum *= __half2float(a.scale[row]);
    if (a.bias) sum += __half2float(a.bias[row]);
    if (j < nvalid) {
      const int64_t o = TM ? (n0 + j) * a.m + row : row * a.n + n0 + j;
      if constexpr (sizeof(OutT) == 2) static_cast<__half*>(a.d)[o] = __float2half_rn(sum);
      else static_cast<float*>(a.d)[o] = sum;
    }
  }
  OB_TRACE_EV(7);
}

template <int NT, typename OutT, bool TM>
cudaError_t launch(const DecodeArgs& a, int S, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(a.m / 128), (unsigned)S, (unsigned)((a.n + NT * 8 - 1) / (NT * 8)));
  cfg.blockDim = dim3(512);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)S;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, ob_gemm_decode_kernel<NT, OutT, TM>, a);
}

}  // namespace

namespace ob {

namespace {
int pick_split(int64_t m, int64_t k) {
  // split K over a cluster of up to 8 CTAs (16 slices), as far as there are tiles and until the
  // grid holds about two CTAs per SM
  const int64_t tiles_k = k / OB_TILE_K, row_blocks = m / 128;
  int S = 1;
  while (S < 8 && 4 * S <= tiles_k && row_blocks * S < 2 * 148) S *= 2;
  // tuning knob for experiments
  static const int forced = [] { const char* v = getenv("ONEBIT_DECODE_SPLIT"); return v ? atoi(v) : 0; }();
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) S = forced;
  return S;
}
template <bool TM>
cudaError_t dispatch(const DecodeArgs& a, int out_type, cudaStream_t stream) {
  const int S = pick_split(a.m, a.k);
  const bool two = (a.n > 8);
  if (out_type == OB_OUT_F16) return two ? launch<2, __half, TM>(a, S, stream) : launch<1, __half, TM>(a, S, stream);
  return two ? launch<2, float, TM>(a, S, stream) : launch<1, float, TM>(a, S, stream);
}
}  // namespace

cudaError_t launch_gemm_decode(const void* bits_tile, const void* meta_tile, const void* scale, const void* b,
                               void* d, int64_t m, int64_t n, int64_t k, int out_type, cudaStream_t stream) {
  DecodeArgs a{static_cast<const uint8_t*>(bits_tile), static_cast<const uint8_t*>(meta_tile),
               static_cast<const __half*>(scale), nullptr, static_cast<const __half*>(b), d, m, n, k};
  return dispatch<false>(a, out_type, stream);
}

cudaError_t launch_gemm_decode_tokens(const void* bits_tile, const void* meta_tile, const void* scale, const void* bias,
                                      const void* x, void* y, int64_t m, int64_t n, int64_t k, int out_type,
                                      cudaStream_t stream) {
  DecodeArgs a{static_cast<const uint8_t*>(bits_tile), static_cast<const uint8_t*>(meta_tile),
               static_cast<const __half*>(scale), static_cast<const __half*>(bias), static_cast<const __half*>(x), y, m, n, k};
  return dispatch<true>(a, out_type, stream);
}

}  // namespace ob

#ifdef OB_TRACE
extern "C" int onebit_debug_read_trace_decode(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_trace_dec, sizeof(long long) * 4 * 16);
}
#endif
