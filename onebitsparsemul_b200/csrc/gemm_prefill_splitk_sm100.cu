// K2, split-K form: the tensor-memory kernel for the shapes between the regimes (tens to a few hundred tokens
// on 7B-class layers), where the output has too few 128 x 128 tiles to fill the chip and one CTA per tile would
// walk the whole k loop alone (the reference launches (m/128, n/64) CTAs with split_k_slices = 1 for them,
// csrc/kernel.h:23, csrc/kernel_lib.cu:62).
//
// Same pipeline as the single-CTA kernel of gemm_prefill_sm100.cu (TMA producer, expander warps writing the +-1
// operand to tensor memory, one MMA thread, tcgen05.mma.sp with M = 128, N = 128, K = 32) on ONE SLICE of k: a
// cluster of S CTAs along z shares an output tile. At the end every CTA holds a 128 x 128 fp32 partial tile in
// tensor memory; each of its rows goes, as asynchronous 16-byte stores that complete on the receiver's mbarrier
// (st.async), into a dedicated shared-memory buffer of the CTA that owns the row -- CTA o of the cluster owns
// rows [o * ceil(128 / S), ...) -- which adds the S slices in a fixed order, scales, converts and stores. No
// scratch in global memory, no atomics, deterministic. The receive buffer is separate from the pipeline stages:
// a fast CTA pushes while a slow one still multiplies.
// No TMA load uses cluster multicast. Every mbarrier wait is bounded (see sm100_ptx.h).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <cstdlib>

#include "formats.h"
#include "kernels.h"
#include "sm100_ptx.h"

namespace {

using namespace ob_ptx;

constexpr int BM = 128, BK = 128, BN = 128;
constexpr int kStages = 4;
constexpr int kBBoxBytes = BK * 128;                     // 128 k-rows x 64 tokens x 2 B
constexpr int kBBytes = (BN / 64) * kBBoxBytes;          // 32 KiB
constexpr int kStageBytes = kBBytes + OB_TILE_META_BYTES + OB_TILE_BITS_BYTES;
constexpr int kRecvRows = 136;                           // S x ceil(128 / S) <= 133 for S <= 8
constexpr int kRecvBytes = kRecvRows * BN * 4;
constexpr int kSmemBytes = kStages * kStageBytes + kRecvBytes + 1024 /*alignment*/ + 512 /*barriers*/;
constexpr int kThreads = 32 * (2 + 4 + 4);               // producer, MMA, expanders, epilogue
constexpr int kAccCols = BN, kECols = 8, kASlotCols = 32;
constexpr int kTmemCols = 512;                           // 128 accumulator + 8 metadata + 4 x 32 operand slots, rounded up
static_assert(kSmemBytes <= 227 * 1024, "stages and receive buffer exceed shared memory");
static_assert(kAccCols + kECols + kStages * kASlotCols <= 512, "tensor memory exceeded");

struct SplitKArgs {
  const uint8_t* bits_tile;
  const uint8_t* meta_tile;
  const __half* scale;
  void* d;
  int64_t m, n, k;
  int out_type;
  int* status;
};

__device__ __forceinline__ void st_async_v4(uint32_t cluster_addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w, uint32_t cluster_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(cluster_addr), "r"(x), "r"(y), "r"(z), "r"(w), "r"(cluster_bar) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
ob_gemm_prefill_splitk_kernel(const __grid_constant__ CUtensorMap tmap_b, SplitKArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  // stage s: [B 2 x 16 KiB][meta 2 KiB][bits 1 KiB]; then the receive buffer; then the barriers
  auto stage_b = [&](int s) { return smem_base + s * kStageBytes; };
  auto stage_e = [&](int s) { return stage_b(s) + kBBytes; };
  auto stage_bits = [&](int s) { return stage_b(s) + kBBytes + OB_TILE_META_BYTES; };
  const uint32_t recv = smem_base + kStages * kStageBytes;
  const float* recv_gen = reinterpret_cast<const float*>(smem_gen + kStages * kStageBytes);
  const uint32_t bar_base = recv + kRecvBytes;
  auto bar_full = [&](int s) { return bar_base + 8 * s; };                        // TMA landed
  auto bar_empty = [&](int s) { return bar_base + 8 * (kStages + s); };           // MMAs of the stage done (stage and operand slot free)
  auto bar_afull = [&](int s) { return bar_base + 8 * (2 * kStages + s); };       // +-1 values written to slot s
  const uint32_t bar_acc = bar_base + 8 * (3 * kStages);
  const uint32_t bar_recv = bar_acc + 8;                                          // every slice's rows for this CTA have landed
  const uint32_t tmem_slot = bar_recv + 8;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = (int)gridDim.z, rank = (int)blockIdx.z;       // the cluster spans z
  const int64_t mb = blockIdx.x;
  const int64_t n0 = (int64_t)blockIdx.y * BN;
  const int kt_all = (int)(a.k / BK);
  const int kb0 = (int)((int64_t)kt_all * rank / S), kb1 = (int)((int64_t)kt_all * (rank + 1) / S);
  const int kt = kb1 - kb0;                                   // weight tiles of this CTA's slice (>= 1)
  const int rows_per = (BM + S - 1) / S;
  const int rows_owned = max(0, min(rows_per, BM - rank * rows_per));
  long long budget = 2000000000ll;                            // cycles, about a second

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); mbar_init(bar_afull(s), 4); }
    mbar_init(bar_acc, 1);
    mbar_init(bar_recv, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
    if (S > 1) mbar_expect_tx(bar_recv, (uint32_t)(S * rows_owned * BN * 4));
  }
  if (warp == 1) tcgen05_alloc(tmem_slot, kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  // every CTA of the cluster announces that it runs and that its barriers exist; the matching wait stands right
  // before the first store into another CTA's shared memory
  if (S > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_gen;
  const uint32_t tmem_acc = tmem_base, tmem_e = tmem_base + kAccCols, tmem_a = tmem_base + kAccCols + kECols;

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      for (int it = 0; it < kt; ++it) {
        const int s = it % kStages;
        mbar_wait(bar_empty(s), ((it / kStages) & 1) ^ 1, budget, a.status, 1);
        mbar_expect_tx(bar_full(s), kStageBytes);
#pragma unroll
        for (int j = 0; j < BN / 64; ++j)
          tma_load_2d(stage_b(s) + j * kBBoxBytes, &tmap_b, (int)(n0 + 64 * j), (kb0 + it) * BK, bar_full(s));
        const int64_t tile = mb * kt_all + kb0 + it;
        bulk_load(stage_e(s), a.meta_tile + tile * OB_TILE_META_BYTES, OB_TILE_META_BYTES, bar_full(s));
        bulk_load(stage_bits(s), a.bits_tile + tile * OB_TILE_BITS_BYTES, OB_TILE_BITS_BYTES, bar_full(s));
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 2) /*sparse*/ | (1u << 4) /*fp32 accumulate*/ | (1u << 16) /*B is n-major*/ |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      for (int it = 0; it < kt; ++it) {
        const int s = it % kStages;
        mbar_wait(bar_afull(s), (it / kStages) & 1, budget, a.status, 3);   // covers "TMA landed": the expanders waited for it
        tcgen05_fence_after();
        const uint64_t bdesc = make_desc(stage_b(s), kBBoxBytes, 1024, kLayoutSw128);
        const uint32_t e_col = tmem_e + 4 * (it & 1);
        tcgen05_cp_128x128b(e_col, make_desc(stage_e(s), 128, 128, kLayoutNone));
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
          tcgen05_mma_sp_f16_ts(tmem_acc, tmem_a + s * kASlotCols + 8 * kb, bdesc + (uint64_t)(256 * kb), e_col + (kb & ~1),
                                idesc | (uint32_t)(kb & 1), (it | kb) != 0);
        tcgen05_commit(bar_empty(s));
      }
      tcgen05_commit(bar_acc);
    }
  } else if (warp < 6) {
    // ---------------- expander: thread = weight row; the warp's TMEM quadrant is warp % 4 ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;
    for (int it = 0; it < kt; ++it) {
      const int s = it % kStages;
      // the stage landing again implies that the MMAs of its previous use are done: operand slot s is free too
      mbar_wait(bar_full(s), (it / kStages) & 1, budget, a.status, 4);
      __syncwarp();
      const uint2 w = *reinterpret_cast<const uint2*>(smem_gen + (stage_bits(s) - smem_base) + r * 8);
      uint32_t v[32];
#pragma unroll
      for (int j = 0; j < 16; ++j) { v[j] = expand_pair(w.x, j); v[16 + j] = expand_pair(w.y, j); }
      tcgen05_fence_after();
      tcgen05_st_32x32b_x32(tmem_a + ((uint32_t)(q * 32) << 16) + (uint32_t)(s * kASlotCols), v);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_afull(s));
    }
  } else {
    // ---------------- epilogue: warp quadrant = warp % 4, thread = output row ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;
    mbar_wait(bar_acc, 0, budget, a.status, 5);
    __syncwarp();
    tcgen05_fence_after();
    if (S == 1) {
      const int64_t row = mb * BM + r;
      const float sc = a.scale ? __half2float(a.scale[row]) : 1.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tcgen05_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        const int64_t col = n0 + c0;
        if (col >= a.n) continue;
        if (a.out_type == OB_OUT_F16) {
          __half* dst = static_cast<__half*>(a.d) + row * a.n + col;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (col + 8 * j < a.n) {
              uint4 o;
              uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                const __half2 p = __floats2half2_rn(__uint_as_float(v[8 * j + 2 * h]) * sc, __uint_as_float(v[8 * j + 2 * h + 1]) * sc);
                ow[h] = *reinterpret_cast<const uint32_t*>(&p);
              }
              *reinterpret_cast<uint4*>(dst + 8 * j) = o;
            }
          }
        } else {
          float* dst = static_cast<float*>(a.d) + row * a.n + col;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (col + 4 * j < a.n)
              *reinterpret_cast<float4*>(dst + 4 * j) = make_float4(__uint_as_float(v[4 * j]) * sc, __uint_as_float(v[4 * j + 1]) * sc,
                                                                    __uint_as_float(v[4 * j + 2]) * sc, __uint_as_float(v[4 * j + 3]) * sc);
        }
      }
    } else {
      // all CTAs of the cluster have started and initialised their barriers
      asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
      const uint32_t owner = (uint32_t)(r / rows_per);
      const uint32_t dst = map_to_cta(recv + (uint32_t)((rank * rows_per + r % rows_per) * BN * 4), owner);
      const uint32_t dbar = map_to_cta(bar_recv, owner);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tcgen05_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) st_async_v4(dst + (uint32_t)((c0 + 4 * j) * 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3], dbar);
      }
    }
    tcgen05_fence_before();
  }
  __syncwarp();
  if (S > 1) {
    if (warp < 6) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");   // every thread that arrived also waits
    // fixed-order sum of the S slices of this CTA's rows: consecutive threads take consecutive groups of 4 tokens
    mbar_wait(bar_recv, 0, budget, a.status, 6);
    const bool vec16 = a.out_type == OB_OUT_F16 && (reinterpret_cast<uintptr_t>(a.d) & 7) == 0;
    const bool vec32 = a.out_type == OB_OUT_F32 && (reinterpret_cast<uintptr_t>(a.d) & 15) == 0;
    for (int e = threadIdx.x; e < rows_owned * (BN / 4); e += kThreads) {
      const int rr = e / (BN / 4), c = (e % (BN / 4)) * 4;
      const int64_t col = n0 + c;
      if (col >= a.n) continue;                               // n % 8 == 0: a group of 4 is inside or outside
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int sl = 0; sl < S; ++sl) {
        const float4 p = *reinterpret_cast<const float4*>(recv_gen + (size_t)(sl * rows_per + rr) * BN + c);
        sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
      }
      const int64_t row = mb * BM + rank * rows_per + rr;
      const float sc = a.scale ? __half2float(a.scale[row]) : 1.f;
      sum.x *= sc; sum.y *= sc; sum.z *= sc; sum.w *= sc;
      if (a.out_type == OB_OUT_F16) {
        __half* dst = static_cast<__half*>(a.d) + row * a.n + col;
        const __half2 lo = __floats2half2_rn(sum.x, sum.y), hi = __floats2half2_rn(sum.z, sum.w);
        if (vec16) {
          *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        } else {
          dst[0] = __low2half(lo); dst[1] = __high2half(lo); dst[2] = __low2half(hi); dst[3] = __high2half(hi);
        }
      } else {
        float* dst = static_cast<float*>(a.d) + row * a.n + col;
        if (vec32) *reinterpret_cast<float4*>(dst) = sum;
        else { dst[0] = sum.x; dst[1] = sum.y; dst[2] = sum.z; dst[3] = sum.w; }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tcgen05_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

namespace ob {

// K slices for a problem of `tiles` output tiles (128 x 128) and kt weight tiles along k. Measured with CUDA-graph
// replays: a CTA of this kernel walks a weight tile in ~800 cycles, starts up in ~3 000, and the hand-off of the
// 64 KiB partial tiles costs ~9 000 (4096 x 4096 with 128 tokens: 15.1 us unsplit, 11.5 us with 4 slices). A split
// only pays while all slices of all tiles run in ONE wave (11008 x 4096 with 256 tokens, 172 tiles: 29 us unsplit,
// 40 us with 2 slices), so larger grids stay unsplit.
int prefill_splitk_choose(int64_t tiles, int64_t kt) {
  const long long sms = sm_count();
  constexpr long long kStart = 3000, kTile = 800, kHandOff = 9000;
  int best = 1;
  long long best_cost = ((tiles + sms - 1) / sms) * (kStart + kt * kTile);
  for (int S = 2; S <= 8; ++S) {
    if (kt < 2 * S || tiles * S > sms) break;
    const long long cost = kStart + ((kt + S - 1) / S) * kTile + kHandOff;
    if (cost < best_cost) { best = S; best_cost = cost; }
  }
  static const int forced = [] { const char* v = getenv("ONEBIT_PREFILL_SPLIT"); return v ? atoi(v) : 0; }();
  if (forced >= 1 && forced <= 8 && 2 * forced <= kt) best = forced;
  return best;
}

// tmap: B (k x n), boxes of 64 tokens x 128 k-rows, 128-byte swizzle
cudaError_t launch_gemm_prefill_splitk(const CUtensorMap* tmap, int S, const void* bits_tile, const void* meta_tile,
                                       const void* scale, void* d, int64_t m, int64_t n, int64_t k, int out_type,
                                       int* status, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(ob_gemm_prefill_splitk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  SplitKArgs a{static_cast<const uint8_t*>(bits_tile), static_cast<const uint8_t*>(meta_tile), static_cast<const __half*>(scale),
               d, m, n, k, out_type, status};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(m / BM), (unsigned)((n + BN - 1) / BN), (unsigned)S);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)S;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, ob_gemm_prefill_splitk_kernel, *tmap, a);
}

}  // namespace ob
