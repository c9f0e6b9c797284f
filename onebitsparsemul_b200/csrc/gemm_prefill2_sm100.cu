// K2, CTA-pair form: the compute-bound kernel with the 2-CTA tensor-core instruction.
//
// Same pipeline as gemm_prefill_sm100.cu (TMA producer, expander warps writing the +-1 operand to
// tensor memory, one MMA thread, epilogue warps) but two CTAs of a cluster share every MMA:
// tcgen05.mma.sp.cta_group::2 with M = 256 (128 weight rows per CTA) and N = 256, where each CTA
// stages only ITS half of the token tile (128 of the 256 tokens). Per flop that halves both the
// tensor core's shared-memory reads and the TMA writes of the token tile -- the shared-memory port
// is what bounds the single-CTA kernel -- and halves the L2 -> SM traffic per SM.
//
// Roles across the pair
//   both CTAs   producer: own token half + own weight tile's metadata / sign blocks -> own stage,
//               own "full" barrier. Expanders: wait own "full" and own operand-slot "empty", write
//               +-1 to own tensor memory, then arrive (one lane per warp) on the LEADER's "operand full"
//               barrier (a remote arrive for the second CTA). That one barrier therefore tells the leader
//               that both CTAs' stage data has landed and both operand slots are written.
//   leader      (cluster rank 0) MMA thread: tcgen05.cp.cta_group::2 of the metadata, 4 MMAs per
//               stage, tcgen05.commit with cluster multicast onto both CTAs' "stage empty",
//               "slot empty" and, at the end, "accumulator full" barriers.
//   both CTAs   epilogue from own tensor memory; a cluster barrier before tensor memory is freed.
// No TMA load uses cluster multicast. Every mbarrier wait is bounded (see sm100_ptx.h).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>

#include "formats.h"
#include "kernels.h"
#include "sm100_ptx.h"

namespace {

using namespace ob_ptx;

// Timeline instrumentation for tuning, compiled in only with -DOB_TRACE (see gemm_prefill_sm100.cu):
// the two CTAs of one pair record the SM clock at every hand-over (events 0-7 leader, 8-15 partner).
#ifdef OB_TRACE
__device__ long long g_trace2[16][512];
#define OB_TRACE_EV(ev, it) do { if ((blockIdx.x >> 1) == 5 && blockIdx.y == 7 && (it) < 512) g_trace2[(ev) + 8 * (blockIdx.x & 1)][it] = clock64(); } while (0)
#else
#define OB_TRACE_EV(ev, it) do { } while (0)
#endif

constexpr int BM = 128;              // weight rows per CTA
constexpr int BK = 128;              // dense k per stage
constexpr int BN = 256;              // tokens per CTA pair
constexpr int BNH = BN / 2;          // tokens staged per CTA
constexpr int NXG = 1;               // expander groups of 4 warps

// KS = weight tiles (128 dense k each) per pipeline stage. Two tiles per stage halve the per-stage
// fixed work of the MMA thread (barrier wait, fence, commit) relative to the 8 MMAs it issues.
template <int KS> struct Cfg2 {
  static constexpr int kBBoxBytes = KS * BK * 128;                                         // one 64-token column chunk
  static constexpr int kBBytes = (BNH / 64) * kBBoxBytes;                                  // KS x 32 KiB
  static constexpr int kStageBytes = kBBytes + KS * (OB_TILE_META_BYTES + OB_TILE_BITS_BYTES);
  static constexpr int kStages = (KS == 1) ? 6 : 3;
  static constexpr int kAccCols = BN;              // 256
  static constexpr int kECols = KS * 8;            // per weight tile two 4-column metadata slots
  static constexpr int kASlotCols = KS * 32;
  static constexpr int kASlots = kStages;          // operand slot x = stage x: one barrier frees both
  static constexpr int kTmemCols = 512;            // 256 + 8 KS + 192 used
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 512;
  static constexpr int kThreads = 32 * (2 + 4 * NXG + 4);
  static_assert(kSmemBytes <= 227 * 1024, "stages exceed shared memory");
  static_assert(kAccCols + kECols + kASlots * kASlotCols <= 512, "tensor memory exceeded");
};

struct Prefill2Args {
  const uint8_t* bits_tile;
  const uint8_t* meta_tile;
  const __half* scale;
  const __half* bias;  // per output row, added after the scale (token-major callers; NULL = none)
  void* d;
  int64_t m, n, k;
  int out_type;
  int* status;
  int tma_store;     // 1: fp16 output leaves through shared memory and TMA stores (tmap_c is valid)
  int group;         // token blocks per rasterisation group (see tile_of_cluster)
};

// Which output tile a cluster computes. Clusters are numbered in launch order (row pairs fastest). With the plain
// (row pair, token block) = (x / 2, y) assignment all row pairs of ONE token block run together: the token panel
// (k x 256 fp16) is read from HBM once, but the packed weights are streamed again for every token block -- at
// 25600^3 that is 100 x 123 MB, and ncu measured 13.6 GB of DRAM reads per launch against 1.43 GB of operands. Here
// `group` token blocks are interleaved under one sweep over the row pairs: their panels (sized on the host to about
// half of L2) stay hot while the weights stream past, so the weights are read ceil(blocks / group) times instead
// of once per token block.
__device__ __forceinline__ void tile_of_cluster(int group, int64_t& row_pair, int64_t& token_block) {
  const int64_t pairs = gridDim.x >> 1, blocks = gridDim.y;
  const int64_t lin = (int64_t)blockIdx.y * pairs + (blockIdx.x >> 1);
  const int64_t per_group = pairs * group;
  const int64_t g = lin / per_group, r = lin - g * per_group;
  const int64_t width = min((int64_t)group, blocks - g * group);   // the last group may be narrower
  row_pair = r / width;
  token_block = g * group + (r - row_pair * width);
}

// TM = token-major operands, the nn.Linear convention: tokens x (n, k) row-major, i.e. a K-major B operand,
//      and output y (n, m) row-major, i.e. C transposed. false = the reference's B (k, n), C (m, n).
template <int KS, bool TM>
__global__ void __launch_bounds__(Cfg2<KS>::kThreads, 1)
ob_gemm_prefill2_kernel(const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_c,
                        Prefill2Args a) {
  using C = Cfg2<KS>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  // stage s: [B half: 2 column chunks x (KS*128 k-rows x 128 B)][meta KS x 2 KiB][bits KS x 1 KiB]
  auto stage_b = [&](int s) { return smem_base + s * C::kStageBytes; };
  auto stage_e = [&](int s, int j) { return stage_b(s) + C::kBBytes + j * OB_TILE_META_BYTES; };
  auto stage_bits = [&](int s, int j) { return stage_b(s) + C::kBBytes + KS * OB_TILE_META_BYTES + j * OB_TILE_BITS_BYTES; };
  const uint32_t bar_base = smem_base + C::kStages * C::kStageBytes;
  auto bar_full = [&](int s) { return bar_base + 8 * s; };                                    // own TMA landed
  auto bar_empty = [&](int s) { return bar_base + 8 * (C::kStages + s); };                    // pair's MMAs of the stage done
  auto bar_afull = [&](int x) { return bar_base + 8 * (2 * C::kStages + x); };                // leader only: both CTAs wrote slot x
  const uint32_t bar_acc = bar_base + 8 * (3 * C::kStages);
  const uint32_t tmem_slot = bar_acc + 8;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();           // 0 = leader
  int64_t row_pair, token_block;
  tile_of_cluster(a.group, row_pair, token_block);
  const int64_t mt = 2 * row_pair + cta;            // weight tile of this CTA (pair = tiles 2p, 2p+1)
  const int64_t n0 = token_block * BN + (int64_t)cta * BNH;   // first token this CTA stages
  const int kt = (int)(a.k / BK);                   // weight tiles along k
  const int nit = (kt + KS - 1) / KS;               // pipeline iterations; the last may hold fewer tiles
  long long budget = 2000000000ll;

  // one stage of TMA traffic: own half of the token tile + the weight tiles' metadata and sign blocks
  auto load_stage = [&](int it) {
    const int s = it % C::kStages;
    const int tiles = min(KS, kt - it * KS);
    // token rows past k (odd tile count) are zero-filled by TMA and still count as bytes
    mbar_expect_tx(bar_full(s), C::kBBytes + tiles * (OB_TILE_META_BYTES + OB_TILE_BITS_BYTES));
    if constexpr (TM) {
      // K-major token tile: boxes of 64 k (128 bytes) x 128 tokens, two per weight tile
#pragma unroll
      for (int j = 0; j < 2 * KS; ++j)
        tma_load_2d(stage_b(s) + j * (BNH * 128), &tmap_b, (it * KS * BK) + 64 * j, (int)n0, bar_full(s));
    } else {
#pragma unroll
      for (int j = 0; j < BNH / 64; ++j)
        tma_load_2d(stage_b(s) + j * C::kBBoxBytes, &tmap_b, (int)(n0 + 64 * j), it * KS * BK, bar_full(s));
    }
    for (int j = 0; j < tiles; ++j) {
      const int64_t tile = mt * kt + it * KS + j;
      bulk_load(stage_e(s, j), a.meta_tile + tile * OB_TILE_META_BYTES, OB_TILE_META_BYTES, bar_full(s));
      bulk_load(stage_bits(s, j), a.bits_tile + tile * OB_TILE_BITS_BYTES, OB_TILE_BITS_BYTES, bar_full(s));
    }
  };
  const int npre = min(C::kStages, nit);            // stages filled before anything else happens

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int x = 0; x < C::kASlots; ++x) mbar_init(bar_afull(x), 2 * 4 * NXG);
    mbar_init(bar_acc, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
    if (a.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_c) : "memory");
    // the first ring of loads only needs this CTA's own barriers: start it now, so that its latency
    // overlaps the tensor-memory allocation and the cluster-wide start-up barrier
    for (int it = 0; it < npre; ++it) load_stage(it);
  }
  if (threadIdx.x == 0) OB_TRACE_EV(7, 2);
  if (warp == 1) tcgen05_alloc_2cta(tmem_slot, C::kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                               // both CTAs' barriers exist before any remote arrive
  tcgen05_fence_after();
  if (threadIdx.x == 0) OB_TRACE_EV(7, 4);
  const uint32_t tmem_base = *tmem_slot_gen;
  const uint32_t tmem_acc = tmem_base;
  const uint32_t tmem_e = tmem_base + C::kAccCols;
  const uint32_t tmem_a = tmem_base + C::kAccCols + C::kECols;

  if (warp == 0) {
    // ---------------- producer (both CTAs): the stages after the pre-issued first ring ----------------
    if (lane == 0) {
      for (int it = npre; it < nit; ++it) {
        mbar_wait(bar_empty(it % C::kStages), ((it / C::kStages) & 1) ^ 1, budget, a.status, 1);
        OB_TRACE_EV(0, it);
        load_stage(it);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (cta == 0 && lane == 0) {
      const uint32_t idesc = (1u << 2) /*sparse*/ | (1u << 4) /*fp32 accumulate*/ | (TM ? 0u : (1u << 16)) /*B n-major*/ |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      for (int it = 0; it < nit; ++it) {
        const int s = it % C::kStages, x = s;
        const int tiles = min(KS, kt - it * KS);
        mbar_wait(bar_afull(x), (it / C::kASlots) & 1, budget, a.status, 3);
        OB_TRACE_EV(5, it);
        tcgen05_fence_after();
        const uint64_t bdesc = make_desc(stage_b(s), C::kBBoxBytes, 1024, kLayoutSw128);
#pragma unroll
        for (int j = 0; j < KS; ++j) {
          if (j < tiles) {
            const uint32_t e_col = tmem_e + 8 * j + 4 * (it & 1);
            tcgen05_cp_128x128b_2cta(e_col, make_desc(stage_e(s, j), 128, 128, kLayoutNone));
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
              // token tile of k-block kb of weight tile j: 32 k-rows (4 KiB) further in the n-major form;
              // in the K-major form box 2j + kb/2 (16 KiB each), 64 bytes along its swizzled rows for odd kb
              const uint64_t bd = TM ? make_desc(stage_b(s) + (2 * j + (kb >> 1)) * (BNH * 128) + (kb & 1) * 64, 16, 1024, kLayoutSw128)
                                     : bdesc + (uint64_t)(1024 * j + 256 * kb);
              tcgen05_mma_sp_f16_ts_2cta(tmem_acc, tmem_a + x * C::kASlotCols + 32 * j + 8 * kb, bd, e_col + (kb & ~1),
                                         idesc | (uint32_t)(kb & 1), (it | j | kb) != 0);
            }
          }
        }
        tcgen05_commit_2cta(bar_empty(s), 3);     // frees stage s and operand slot s in both CTAs
        OB_TRACE_EV(6, it);
      }
      tcgen05_commit_2cta(bar_acc, 3);
    }
  } else if (warp < 2 + 4 * NXG) {
    // ---------------- expander (both CTAs): thread = weight row, TMEM quadrant = warp % 4 ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;
    for (int it = 0; it < nit; ++it) {
      // stage s landing again implies that the pair's MMAs of its previous use are done, so operand
      // slot s is free as well
      const int s = it % C::kStages, x = s;
      const int tiles = min(KS, kt - it * KS);
      mbar_wait(bar_full(s), (it / C::kStages) & 1, budget, a.status, 4);
      if (threadIdx.x == 64) OB_TRACE_EV(1, it);
      tcgen05_fence_after();
#pragma unroll
      for (int j = 0; j < KS; ++j) {
        if (j < tiles) {
          const uint2 w = *reinterpret_cast<const uint2*>(smem_gen + (stage_bits(s, j) - smem_base) + r * 8);
          uint32_t v[32];
#pragma unroll
          for (int p = 0; p < 16; ++p) { v[p] = expand_pair(w.x, p); v[16 + p] = expand_pair(w.y, p); }
          tcgen05_st_32x32b_x32(tmem_a + ((uint32_t)(q * 32) << 16) + (uint32_t)(x * C::kASlotCols + 32 * j), v);
        }
      }
      tcgen05_fence_before();
      // one arrive per warp: a remote arrive is a cluster transaction
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_afull(x), 0));
      if (threadIdx.x == 64) OB_TRACE_EV(3, it);
    }
  } else {
    // ---------------- epilogue (both CTAs): own 128 rows x all 256 tokens of the pair ----------------
    const int q = warp & 3;
    mbar_wait(bar_acc, 0, budget, a.status, 5);
    if (q == 0 && lane == 0) OB_TRACE_EV(7, 0);
    tcgen05_fence_after();
    const int64_t row = mt * BM + q * 32 + lane;
    const int64_t nbase = token_block * BN;
    const float sc = a.scale ? __half2float(a.scale[row]) : 1.f;
    const bool has_bias = a.bias != nullptr;
    const float bs = has_bias ? __half2float(a.bias[row]) : 0.f;
    auto fin = [&](uint32_t acc) { const float x = __uint_as_float(acc) * sc; return has_bias ? x + bs : x; };
    if constexpr (TM) {
      // y (n, m) row-major: this thread owns output feature `row`; the 32 accumulator columns of a chunk
      // are 32 tokens, i.e. 32 rows of y
      if (a.tma_store) {
        // fp16: the transposed tile is assembled in the idle first pipeline stage as 2 boxes of
        // 256 tokens x 64 features (128-byte swizzle) and leaves with 2 TMA stores
        uint8_t* cbuf = smem_gen + (stage_b(0) - smem_base);
        const int r = q * 32 + lane;
        uint8_t* mybox = cbuf + (r >> 6) * (BN * 128) + (r & 7) * 2;
        const int chunk = (r & 63) >> 3;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tcgen05_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int t = c0 + j;
            *reinterpret_cast<__half*>(mybox + t * 128 + ((chunk ^ (t & 7)) << 4)) = __float2half_rn(fin(v[j]));
          }
        }
        fence_proxy_async();
        asm volatile("bar.sync 1, 128;" ::: "memory");        // the four epilogue warps
        if (q == 0 && lane == 0) {
#pragma unroll
          for (int bx = 0; bx < 2; ++bx)
            tma_store_2d(&tmap_c, smem_u32(cbuf) + bx * (BN * 128), (int)(mt * BM + 64 * bx), (int)nbase);
          tma_store_commit_and_wait();
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tcgen05_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int64_t t = nbase + c0 + j;
            if (t < a.n) {
              if (a.out_type == OB_OUT_F16) static_cast<__half*>(a.d)[t * a.m + row] = __float2half_rn(fin(v[j]));
              else static_cast<float*>(a.d)[t * a.m + row] = fin(v[j]);
            }
          }
        }
      }
    } else
    if (a.tma_store) {
      // fp16 output: the tile is assembled in the (now idle) first pipeline stage as 4 boxes of
      // 128 rows x 64 tokens with the 128-byte swizzle, then written with 4 TMA stores: full-line
      // writes, and the threads are done as soon as their rows are in shared memory
      uint8_t* cbuf = smem_gen + (stage_b(0) - smem_base);
      const int r = q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tcgen05_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        uint8_t* box_row = cbuf + (c0 >> 6) * (BM * 128) + r * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 o;
          uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const __half2 p = __floats2half2_rn(fin(v[8 * j + 2 * h]), fin(v[8 * j + 2 * h + 1]));
            ow[h] = *reinterpret_cast<const uint32_t*>(&p);
          }
          const int chunk = ((c0 & 63) >> 3) + j;              // 16-byte chunk inside the 128-byte box row
          *reinterpret_cast<uint4*>(box_row + ((chunk ^ (r & 7)) << 4)) = o;
        }
      }
      fence_proxy_async();
      asm volatile("bar.sync 1, 128;" ::: "memory");          // the four epilogue warps
      if (q == 0 && lane == 0) {
#pragma unroll
        for (int bx = 0; bx < BN / 64; ++bx)
          if (nbase + 64 * bx < a.n) tma_store_2d(&tmap_c, smem_u32(cbuf) + bx * (BM * 128), (int)(nbase + 64 * bx), (int)(mt * BM));
        tma_store_commit_and_wait();
      }
    } else {
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
      uint32_t v[32];
      tcgen05_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
      const int64_t col = nbase + c0;
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
              const __half2 p = __floats2half2_rn(fin(v[8 * j + 2 * h]), fin(v[8 * j + 2 * h + 1]));
              ow[h] = *reinterpret_cast<const uint32_t*>(&p);
            }
            *reinterpret_cast<uint4*>(dst + 8 * j) = o;
          }
        }
      } else {
        float* dst = static_cast<float*>(a.d) + row * a.n + col;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (col + 4 * j < a.n) {
            float4 o = make_float4(fin(v[4 * j]), fin(v[4 * j + 1]), fin(v[4 * j + 2]), fin(v[4 * j + 3]));
            *reinterpret_cast<float4*>(dst + 4 * j) = o;
          }
        }
      }
    }
    }
    tcgen05_fence_before();
    if (q == 0 && lane == 0) OB_TRACE_EV(7, 1);
  }

  __syncthreads();
  cluster_sync_all();               // the partner may still signal this CTA's barriers or read its memory
  if (warp == 1) {
    tcgen05_fence_after();
    tcgen05_dealloc_2cta(tmem_base, C::kTmemCols);
  }
}

}  // namespace

namespace ob {

bool prefill2_supported(int64_t m, int64_t n, int64_t k) {
  return m % (2 * BM) == 0 && k % BK == 0 && n % 8 == 0 && n >= 8 && k >= BK;
}

namespace {
template <int KS, bool TM>
cudaError_t launch2(const CUtensorMap& tmap, const CUtensorMap& tmap_c, const Prefill2Args& a, cudaStream_t stream) {
  using C = Cfg2<KS>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(ob_gemm_prefill2_kernel<KS, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(a.m / BM), (unsigned)((a.n + BN - 1) / BN));
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, ob_gemm_prefill2_kernel<KS, TM>, tmap, tmap_c, a);
}
}  // namespace

// tmap:   tensor map of the tokens -- reference form: B (k x n), boxes of 64 tokens x (128 * ks) k-rows;
//         token-major form: x (n x k), boxes of 64 k x 128 tokens; 128-byte swizzle either way
// tmap_c: tensor map of an fp16 output with the 128-byte swizzle -- C (m x n): boxes of 64 tokens x 128 rows;
//         y (n x m): boxes of 64 features x 256 tokens -- or NULL (fp32 output, or an output that is not
//         16-byte aligned): direct stores from registers
// Token blocks (256 tokens) per rasterisation group of the CTA-pair kernels: the group's token panels (k x 256 fp16
// each) should fill about a quarter of L2, so that they stay hot while one sweep over the row pairs streams the
// weights past (measured at 25600^3: 14.19 ms with 1, 13.66 with 2, 13.72 with 4, 13.96 with 6, 14.13 with 8 blocks).
int prefill_raster_group(int64_t m, int64_t k) {
  static int l2_bytes[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && l2_bytes[dev] == 0 && cudaDeviceGetAttribute(&l2_bytes[dev], cudaDevAttrL2CacheSize, dev) != cudaSuccess) l2_bytes[dev] = 0;
  const int64_t l2 = (dev >= 0 && dev < 64 && l2_bytes[dev] > 0) ? l2_bytes[dev] : (64ll << 20);
  static const int forced_group = [] { const char* v = getenv("ONEBIT_PREFILL_GROUP"); return v ? atoi(v) : 0; }();
  int group = (int)std::max<int64_t>(1, std::min<int64_t>(4, (l2 / 4) / (k * BN * 2)));
  // small weights stay in L2 whatever the order: keep the plain order, whose concurrent clusters share one panel
  if (m * k * 3 / 16 <= l2 / 4) group = 1;
  if (forced_group > 0) group = forced_group;
  return group;
}

cudaError_t launch_gemm_prefill2(const CUtensorMap* tmap, const CUtensorMap* tmap_c, int ks, bool token_major,
                                 const void* bits_tile, const void* meta_tile, const void* scale, const void* bias,
                                 void* d, int64_t m, int64_t n, int64_t k, int out_type, int* status,
                                 cudaStream_t stream) {
  const int group = prefill_raster_group(m, k);
  Prefill2Args a{static_cast<const uint8_t*>(bits_tile), static_cast<const uint8_t*>(meta_tile),
                 static_cast<const __half*>(scale), static_cast<const __half*>(bias), d, m, n, k, out_type, status,
                 tmap_c != nullptr, group};
  const CUtensorMap& tc = tmap_c ? *tmap_c : *tmap;          // unused when tma_store == 0
  if (token_major) return ks == 2 ? launch2<2, true>(*tmap, tc, a, stream) : launch2<1, true>(*tmap, tc, a, stream);
  return ks == 2 ? launch2<2, false>(*tmap, tc, a, stream) : launch2<1, false>(*tmap, tc, a, stream);
}

}  // namespace ob

#ifdef OB_TRACE
extern "C" int onebit_debug_read_trace2(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_trace2, sizeof(long long) * 16 * 512);
}
#endif
