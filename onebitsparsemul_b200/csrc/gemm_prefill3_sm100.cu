// K2, persistent CTA-pair form: the kernel for large fp16-output shapes.
//
// Same CTA-pair pipeline as gemm_prefill2_sm100.cu (tcgen05.mma.sp.cta_group::2, M = 256 rows x
// N = 256 tokens per pair, two weight tiles per stage, +-1 operand and metadata in tensor memory),
// but one cluster per SM pair stays resident and walks over its output tiles:
//   * tensor-memory allocation, barrier set-up and the cluster start-up barrier are paid once per SM
//     instead of once per tile;
//   * the stage ring runs straight through tile boundaries: while the epilogue of tile i drains the
//     accumulator, the producer and the expanders already work on tile i+1;
//   * the epilogue first drains its accumulator row into registers as packed fp16 (256 tokens = 128
//     registers), hands the accumulator back to the MMA thread, and only then writes to global
//     memory -- the stores overlap the next tile's main loop. The MMA thread therefore idles only
//     for the drain (~2 000 cycles per tile) instead of prologue + whole epilogue (~7 600).
// Tiles are assigned round-robin over the clusters with the row block running fastest, so the
// clusters working at the same time share token panels in L2.
// No TMA load uses cluster multicast. Every mbarrier wait is bounded (see sm100_ptx.h).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "formats.h"
#include "kernels.h"
#include "sm100_ptx.h"

namespace {

using namespace ob_ptx;

// Timeline instrumentation for tuning, compiled in only with -DOB_TRACE: the two CTAs of one cluster record
// the SM clock per output tile (events 0-7 leader, 8-15 partner).
#ifdef OB_TRACE
__device__ long long g_trace3[16][512];
#define OB_TRACE_EV(ev, it) do { if ((blockIdx.x >> 1) == 5 && (it) < 512) g_trace3[(ev) + 8 * (blockIdx.x & 1)][it] = clock64(); } while (0)
#else
#define OB_TRACE_EV(ev, it) do { } while (0)
#endif

constexpr int BM = 128;              // weight rows per CTA
constexpr int BK = 128;              // dense k per weight tile
constexpr int BN = 256;              // tokens per CTA pair
constexpr int BNH = BN / 2;          // tokens staged per CTA
constexpr int KS = 2;                // weight tiles per pipeline stage

struct Cfg3 {
  static constexpr int kBBoxBytes = KS * BK * 128;                                         // one 64-token column chunk
  static constexpr int kBBytes = (BNH / 64) * kBBoxBytes;                                  // 64 KiB
  static constexpr int kStageBytes = kBBytes + KS * (OB_TILE_META_BYTES + OB_TILE_BITS_BYTES);
  static constexpr int kStages = 3;
  static constexpr int kAccCols = BN;
  static constexpr int kECols = KS * 8;
  static constexpr int kASlotCols = KS * 32;
  static constexpr int kTmemCols = 512;            // 256 + 16 + 192 used
  static constexpr int kEpiBytes = 4 * 2048;       // per epilogue warp: 4 output rows (512 bytes each) in flight
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 512 + kEpiBytes;
  static constexpr int kThreads = 32 * (2 + 4 + 4);   // producer, MMA, 4 expander warps, 4 epilogue warps
  static_assert(kSmemBytes <= 227 * 1024, "stages exceed shared memory");
  static_assert(kAccCols + kECols + kStages * kASlotCols <= 512, "tensor memory exceeded");
};

struct Prefill3Args {
  const uint8_t* bits_tile;
  const uint8_t* meta_tile;
  const __half* scale;
  const __half* bias;      // per output row, added after the scale (NULL = none)
  __half* d[8];           // reference layout: every destination receives the whole result (d[0] = the caller's C)
  int n_dst;
  int64_t m, n, k;
  int row_blocks;          // m / 256
  int total_tiles;         // row_blocks * ceil(n / 256)
  int* status;
};

// TM = token-major operands (x (n, k), y (n, m)); false = the reference's B (k, n), C (m, n)
// MULTI = the result goes to a.n_dst > 1 buffers (reference layout only)
template <bool TM, bool MULTI>
__global__ void __launch_bounds__(Cfg3::kThreads, 1)
ob_gemm_prefill3_kernel(const __grid_constant__ CUtensorMap tmap_b, Prefill3Args a) {
  using C = Cfg3;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  auto stage_b = [&](int s) { return smem_base + s * C::kStageBytes; };
  auto stage_e = [&](int s, int j) { return stage_b(s) + C::kBBytes + j * OB_TILE_META_BYTES; };
  auto stage_bits = [&](int s, int j) { return stage_b(s) + C::kBBytes + KS * OB_TILE_META_BYTES + j * OB_TILE_BITS_BYTES; };
  const uint32_t bar_base = smem_base + C::kStages * C::kStageBytes;
  auto bar_full = [&](int s) { return bar_base + 8 * s; };                       // own TMA landed
  auto bar_empty = [&](int s) { return bar_base + 8 * (C::kStages + s); };       // pair's MMAs of the stage done
  auto bar_afull = [&](int s) { return bar_base + 8 * (2 * C::kStages + s); };   // leader only: both CTAs wrote slot s
  const uint32_t bar_acc_full = bar_base + 8 * (3 * C::kStages);                 // a tile's MMAs are done
  const uint32_t bar_acc_empty = bar_acc_full + 8;                               // leader only: both CTAs drained the accumulator
  const uint32_t tmem_slot = bar_acc_empty + 8;
  const uint32_t epi_buf = bar_base + 512;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();                      // 0 = leader
  const int cluster_id = (int)(blockIdx.x >> 1), num_clusters = (int)(gridDim.x >> 1);
  const int kt = (int)(a.k / BK);
  const int nit = (kt + KS - 1) / KS;                          // pipeline iterations per tile
  const int my_tiles = (a.total_tiles - cluster_id + num_clusters - 1) / num_clusters;
  const int total_its = my_tiles * nit;                        // the ring runs through all of them
  long long budget = 2000000000ll;

  // iteration gi of this cluster -> (tile coordinates, k position)
  auto tile_of = [&](int gi, int& pb, int& nb, int& it) {
    const int tl = gi / nit;
    it = gi - tl * nit;
    const int t = cluster_id + tl * num_clusters;
    nb = t / a.row_blocks;
    pb = t - nb * a.row_blocks;
  };
  auto load_stage = [&](int gi) {
    int pb, nb, it;
    tile_of(gi, pb, nb, it);
    const int s = gi % C::kStages;
    const int tiles = min(KS, kt - it * KS);
    const int64_t mt = (int64_t)pb * 2 + cta;                  // this CTA's weight tile row
    const int n0 = nb * BN + (int)cta * BNH;                   // first token this CTA stages
    mbar_expect_tx(bar_full(s), C::kBBytes + tiles * (OB_TILE_META_BYTES + OB_TILE_BITS_BYTES));
    if constexpr (TM) {
#pragma unroll
      for (int j = 0; j < 2 * KS; ++j)
        tma_load_2d(stage_b(s) + j * (BNH * 128), &tmap_b, (it * KS * BK) + 64 * j, n0, bar_full(s));
    } else {
#pragma unroll
      for (int j = 0; j < BNH / 64; ++j)
        tma_load_2d(stage_b(s) + j * C::kBBoxBytes, &tmap_b, n0 + 64 * j, it * KS * BK, bar_full(s));
    }
    for (int j = 0; j < tiles; ++j) {
      const int64_t tile = mt * kt + it * KS + j;
      bulk_load(stage_e(s, j), a.meta_tile + tile * OB_TILE_META_BYTES, OB_TILE_META_BYTES, bar_full(s));
      bulk_load(stage_bits(s, j), a.bits_tile + tile * OB_TILE_BITS_BYTES, OB_TILE_BITS_BYTES, bar_full(s));
    }
  };
  const int npre = min(C::kStages, total_its);

  if (threadIdx.x == 0) OB_TRACE_EV(7, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); mbar_init(bar_afull(s), 2 * 4); }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 2 * 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
    for (int gi = 0; gi < npre; ++gi) load_stage(gi);          // first ring: only needs this CTA's own barriers
  }
  if (warp == 1) tcgen05_alloc_2cta(tmem_slot, C::kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                                          // both CTAs' barriers exist before any remote arrive
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;
  const uint32_t tmem_acc = tmem_base;
  const uint32_t tmem_e = tmem_base + C::kAccCols;
  const uint32_t tmem_a = tmem_base + C::kAccCols + C::kECols;

  if (warp == 0) {
    // ---------------- producer (both CTAs) ----------------
    if (lane == 0) {
      for (int gi = npre; gi < total_its; ++gi) {
        mbar_wait(bar_empty(gi % C::kStages), ((gi / C::kStages) & 1) ^ 1, budget, a.status, 1);
        load_stage(gi);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (cta == 0 && lane == 0) {
      const uint32_t idesc = (1u << 2) /*sparse*/ | (1u << 4) /*fp32 accumulate*/ | (TM ? 0u : (1u << 16)) /*B n-major*/ |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      int gi = 0;
      for (int tl = 0; tl < my_tiles; ++tl) {
        // the accumulator of the previous tile must have been drained by both CTAs' epilogues
        if (tl > 0) { mbar_wait(bar_acc_empty, (tl - 1) & 1, budget, a.status, 7); tcgen05_fence_after(); }
        OB_TRACE_EV(0, tl);
        for (int it = 0; it < nit; ++it, ++gi) {
          const int s = gi % C::kStages;
          const int tiles = min(KS, kt - it * KS);
          mbar_wait(bar_afull(s), (gi / C::kStages) & 1, budget, a.status, 3);
          tcgen05_fence_after();
          const uint64_t bdesc = make_desc(stage_b(s), C::kBBoxBytes, 1024, kLayoutSw128);
#pragma unroll
          for (int j = 0; j < KS; ++j) {
            if (j < tiles) {
              const uint32_t e_col = tmem_e + 8 * j + 4 * (gi & 1);
              tcgen05_cp_128x128b_2cta(e_col, make_desc(stage_e(s, j), 128, 128, kLayoutNone));
#pragma unroll
              for (int kb = 0; kb < 4; ++kb) {
                const uint64_t bd = TM ? make_desc(stage_b(s) + (2 * j + (kb >> 1)) * (BNH * 128) + (kb & 1) * 64, 16, 1024, kLayoutSw128)
                                       : bdesc + (uint64_t)(1024 * j + 256 * kb);
                tcgen05_mma_sp_f16_ts_2cta(tmem_acc, tmem_a + s * C::kASlotCols + 32 * j + 8 * kb, bd, e_col + (kb & ~1),
                                           idesc | (uint32_t)(kb & 1), (it | j | kb) != 0);
              }
            }
          }
          tcgen05_commit_2cta(bar_empty(s), 3);                // frees stage s and operand slot s in both CTAs
        }
        tcgen05_commit_2cta(bar_acc_full, 3);
        OB_TRACE_EV(1, tl);
      }
    }
  } else if (warp < 6) {
    // ---------------- expander (both CTAs): thread = weight row, TMEM quadrant = warp % 4 ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;
    for (int gi = 0; gi < total_its; ++gi) {
      const int s = gi % C::kStages;
      const int it = gi % nit;
      const int tiles = min(KS, kt - it * KS);
      mbar_wait(bar_full(s), (gi / C::kStages) & 1, budget, a.status, 4);
      tcgen05_fence_after();
#pragma unroll
      for (int j = 0; j < KS; ++j) {
        if (j < tiles) {
          const uint2 w = *reinterpret_cast<const uint2*>(smem_gen + (stage_bits(s, j) - smem_base) + r * 8);
          uint32_t v[32];
#pragma unroll
          for (int p = 0; p < 16; ++p) { v[p] = expand_pair(w.x, p); v[16 + p] = expand_pair(w.y, p); }
          tcgen05_st_32x32b_x32(tmem_a + ((uint32_t)(q * 32) << 16) + (uint32_t)(s * C::kASlotCols + 32 * j), v);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_afull(s), 0));
    }
  } else {
    // ---------------- epilogue (both CTAs): own 128 rows x the 256 tokens of the tile ----------------
    const int q = warp & 3;
    for (int tl = 0; tl < my_tiles; ++tl) {
      int pb, nb, it0;
      tile_of(tl * nit, pb, nb, it0);
      const int64_t row = ((int64_t)pb * 2 + cta) * BM + q * 32 + lane;
      const int64_t nbase = (int64_t)nb * BN;
      const float sc = a.scale ? __half2float(a.scale[row]) : 1.f;
      const bool has_bias = a.bias != nullptr;
      const float bs = has_bias ? __half2float(a.bias[row]) : 0.f;
      mbar_wait(bar_acc_full, tl & 1, budget, a.status, 5);
      if (q == 0 && lane == 0) OB_TRACE_EV(2, tl);
      tcgen05_fence_after();
      // drain: the whole accumulator row as packed fp16 in registers
      uint32_t h[BN / 2];
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tcgen05_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float x0 = __uint_as_float(v[2 * j]) * sc, x1 = __uint_as_float(v[2 * j + 1]) * sc;
          if (has_bias) { x0 += bs; x1 += bs; }
          const __half2 p = __floats2half2_rn(x0, x1);
          h[c0 / 2 + j] = *reinterpret_cast<const uint32_t*>(&p);
        }
      }
      // hand the accumulator back: the next tile's MMAs may start now
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_acc_empty, 0));
      if (q == 0 && lane == 0) OB_TRACE_EV(3, tl);
      // stores, overlapped with the next tile's main loop
      if constexpr (TM) {
#pragma unroll
        for (int j = 0; j < BN / 2; ++j) {
          const int64_t t0 = nbase + 2 * j;
          const __half2 p = *reinterpret_cast<const __half2*>(&h[j]);
          if (t0 < a.n) a.d[0][t0 * a.m + row] = __low2half(p);
          if (t0 + 1 < a.n) a.d[0][(t0 + 1) * a.m + row] = __high2half(p);
        }
      } else if constexpr (!MULTI) {
        // Reference layout, one destination: 16-byte stores straight from the registers (a thread owns a
        // row). Nothing here touches shared memory, whose port the main loop saturates: a staged epilogue
        // took 13 000 cycles per tile, which a short k loop cannot hide.
        __half* dst = a.d[0] + row * a.n + nbase;
#pragma unroll
        for (int j = 0; j < BN / 8; ++j)
          if (nbase + 8 * j < a.n) *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
      } else {
        // Reference layout, several destinations (C itself and, for a row-sharded GEMM whose result every
        // GPU needs, the same rows of the peers' C over NVLink). What crosses the link must be long
        // contiguous runs: with 7 peer destinations, 16-byte pieces of 32 different rows per instruction
        // took 10.3 ms for a 3328 x 25600 x 25600 slab, 64-byte segments 3.2 ms, whole 512-byte rows 2.4 ms
        // (the GEMM alone: 1.5 ms). So the warp passes four of its rows at a time through its own 2 KiB of
        // shared memory: the four owner lanes write their rows (16-byte chunks XOR-swizzled by the row, so
        // the four lanes hit different banks), then every instruction stores one whole row, 32 lanes x 16
        // bytes, to each destination.
        uint8_t* wbuf = smem_gen + (epi_buf - smem_base) + q * 2048;
        const int64_t row_base = ((int64_t)pb * 2 + cta) * BM + q * 32;
#pragma unroll 1
        for (int g4 = 0; g4 < 8; ++g4) {
          if ((lane >> 2) == g4) {
            uint8_t* myrow = wbuf + (lane & 3) * 512;
#pragma unroll
            for (int j = 0; j < BN / 8; ++j)
              *reinterpret_cast<uint4*>(myrow + ((j ^ (lane & 3)) << 4)) = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
          }
          __syncwarp();
#pragma unroll
          for (int ri = 0; ri < 4; ++ri) {
            const uint4 v = *reinterpret_cast<const uint4*>(wbuf + ri * 512 + ((lane ^ ri) << 4));
            const int64_t col = nbase + lane * 8;
            if (col < a.n) {
              const int64_t off = (row_base + 4 * g4 + ri) * a.n + col;
              for (int e = 0; e < a.n_dst; ++e) *reinterpret_cast<uint4*>(a.d[e] + off) = v;
            }
          }
          __syncwarp();
        }
      }
      if (q == 0 && lane == 0) OB_TRACE_EV(4, tl);
    }
  }

  if (threadIdx.x == 0) OB_TRACE_EV(7, 1);
  __syncthreads();
  cluster_sync_all();               // the partner may still signal this CTA's barriers or read its memory
  if (warp == 1) {
    tcgen05_fence_after();
    tcgen05_dealloc_2cta(tmem_base, C::kTmemCols);
  }
}

template <bool TM, bool MULTI>
cudaError_t launch3(const CUtensorMap& tmap, const Prefill3Args& a, cudaStream_t stream) {
  using C = Cfg3;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(ob_gemm_prefill3_kernel<TM, MULTI>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int sms = ob::sm_count();
  const int clusters = std::min(a.total_tiles, std::max(1, sms / 2));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * clusters));
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
  return cudaLaunchKernelEx(&cfg, ob_gemm_prefill3_kernel<TM, MULTI>, tmap, a);
}

}  // namespace

namespace ob {

// fp16 output only (the drained tile lives in registers as packed fp16); d must be 16-byte aligned in
// the reference layout. tmap as for launch_gemm_prefill2 with two weight tiles per stage. extra_dst: up to
// 7 more buffers of the shape of d (reference layout only) that receive the same result, e.g. the peers'
// copies of C in a row-sharded GEMM.
bool prefill3_supported(int64_t m, int64_t n, int64_t k, int out_type, const void* d, bool token_major) {
  return m % (2 * BM) == 0 && k % BK == 0 && k >= BK && n >= 1 && out_type == OB_OUT_F16 &&
         (token_major || (n % 8 == 0 && (reinterpret_cast<uintptr_t>(d) & 15) == 0)) &&
         (m / (2 * BM)) * ((n + BN - 1) / BN) < (1ll << 30);
}

cudaError_t launch_gemm_prefill3(const CUtensorMap* tmap, bool token_major, const void* bits_tile, const void* meta_tile,
                                 const void* scale, const void* bias, void* d, void* const* extra_dst, int n_extra,
                                 int64_t m, int64_t n, int64_t k, int* status, cudaStream_t stream) {
  if (n_extra < 0 || n_extra > 7 || (n_extra > 0 && token_major)) return cudaErrorInvalidValue;
  Prefill3Args a{};
  a.bits_tile = static_cast<const uint8_t*>(bits_tile);
  a.meta_tile = static_cast<const uint8_t*>(meta_tile);
  a.scale = static_cast<const __half*>(scale);
  a.bias = static_cast<const __half*>(bias);
  a.d[0] = static_cast<__half*>(d);
  for (int e = 0; e < n_extra; ++e) {
    if ((reinterpret_cast<uintptr_t>(extra_dst[e]) & 15) != 0) return cudaErrorMisalignedAddress;
    a.d[1 + e] = static_cast<__half*>(extra_dst[e]);
  }
  a.n_dst = 1 + n_extra;
  a.m = m; a.n = n; a.k = k;
  a.row_blocks = (int)(m / (2 * BM));
  a.total_tiles = (int)((m / (2 * BM)) * ((n + BN - 1) / BN));
  a.status = status;
  if (token_major) return launch3<true, false>(*tmap, a, stream);
  return a.n_dst > 1 ? launch3<false, true>(*tmap, a, stream) : launch3<false, false>(*tmap, a, stream);
}

}  // namespace ob

#ifdef OB_TRACE
extern "C" int onebit_debug_read_trace3(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_trace3, sizeof(long long) * 16 * 512);
}
#endif
