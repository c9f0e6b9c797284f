// K2: the compute-bound kernel (prefill / square shapes) on the 5th-generation tensor cores.
//
// Replaces the reference's CUTLASS SparseGemm instantiation (csrc/kernel.h:13-72, threadblock.h,
// warp.h: cp.async multistage + warp-level mma.sp m16n8k32) with a hand-written sm_100a kernel:
//
//   producer warp   TMA: the fp16 token tile B (k x n row-major, 128-byte swizzle) through a tensor
//                   map, and the tile-ordered sign bits (1 KiB) and metadata (2 KiB) of the
//                   128x128 weight tile as plain bulk copies; one mbarrier transaction per stage
//   expander warps  thread = weight row: 64 sign bits -> 64 exact fp16 +-1 values (one shift and
//                   one logic op per pair), stored with tcgen05.st into a ring of tensor-memory
//                   slots (or, in the shared-memory form, K-major with the 128-byte swizzle)
//   MMA thread      tcgen05.cp moves the metadata block into 4 tensor-memory columns, then
//                   4 x tcgen05.mma.sp.kind::f16 (M=128, N=BN, K=32 dense) per weight tile and stage
//                   with the +-1 operand read from tensor memory, fp32 accumulators in tensor
//                   memory; tcgen05.commit frees the stage and the operand slot
//   epilogue warps  tcgen05.ld -> per-row scale -> fp16 / fp32 -> 16-byte global stores
//
// Every wait on an mbarrier is bounded: after ~1 s a thread records a code in the status word and
// carries on without waiting, so the kernel always terminates and releases its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "formats.h"
#include "kernels.h"
#include "sm100_ptx.h"

namespace {

constexpr int BM = 128;             // weight rows per MMA (one weight tile)
constexpr int BK = 128;             // dense k per stage = one weight tile

// MS  = weight tiles (128 rows each) stacked per CTA: the token tile in shared memory is reused by MS
//       MMAs, which divides the L2 -> SM traffic per flop by MS (the weight stream is almost free)
// BN  = tokens per CTA
// NXG = expander groups of 4 warps; group g expands the (stage, tile) items with item % NXG == g, so
//       that the proxy fence and barrier latency of one item overlaps the next item's work
// AT  = where the expanded +-1 operand lives: false = shared memory (K-major, 128-byte swizzle),
//       true = tensor memory (tcgen05.st by the expander, A-from-TMEM form of the MMA). The TMEM
//       form takes the A operand off the shared-memory port entirely (no expander writes, no MMA
//       reads), which is the port this kernel saturates first.
template <int MS, int BN, int NXG, bool AT> struct Cfg {
  static constexpr int kABytes = AT ? 0 : BM * 128;        // 128 rows x 64 fp16, per weight tile
  static constexpr int kBBoxBytes = BK * 128;              // 128 k-rows x 64 tokens x 2 B
  static constexpr int kBBytes = (BN / 64) * kBBoxBytes;
  static constexpr int kStageBytes = MS * (kABytes + OB_TILE_META_BYTES + OB_TILE_BITS_BYTES) + kBBytes;
  static constexpr int kStagesFit = (227 * 1024 - 2048) / kStageBytes;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
  static constexpr int kTxBytes = kBBytes + MS * (OB_TILE_META_BYTES + OB_TILE_BITS_BYTES);
  static constexpr int kAccCols = MS * BN;
  static constexpr int kECols = MS * 8;                    // per weight tile two 4-column metadata slots
  static constexpr int kASlotCols = MS * 32;               // TMEM form: 64 fp16 per row and weight tile
  static constexpr int kASlotsFit = AT ? (512 - kAccCols - kECols) / kASlotCols : 0;
  // ring of +-1 operand slots: the stages themselves (smem form), or TMEM slots -- one per stage if
  // tensor memory has room (then "stage empty" frees both), else a shorter ring of their own
  static constexpr int kASlots = AT ? (kASlotsFit >= kStages ? kStages : kASlotsFit) : kStages;
  static constexpr bool kOwnSlotRing = AT && (kASlots != kStages);
  static constexpr int kUsedCols = kAccCols + kECols + (AT ? kASlots * kASlotCols : 0);
  static constexpr int kTmemCols = kUsedCols <= 128 ? 128 : kUsedCols <= 256 ? 256 : 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 512 /*barriers*/;
  static constexpr int kThreads = 32 * (2 + 4 * NXG + 4);   // producer, MMA, expanders, epilogue
  static_assert(kUsedCols <= 512, "accumulators, metadata and operand slots exceed tensor memory");
  static_assert(kStages >= 2 && kASlots >= 2, "at least two stages and two operand slots");
};

struct PrefillArgs {
  const uint8_t* bits_tile;
  const uint8_t* meta_tile;
  const __half* scale;
  void* d;
  int64_t m, n, k;
  int out_type;
  int* status;
};

using namespace ob_ptx;

// Timeline instrumentation for tuning, compiled in only with -DOB_TRACE: one CTA in the middle of the
// grid records the SM clock at every hand-over of the pipeline.
#ifdef OB_TRACE
__device__ long long g_trace[8][512];
#define OB_TRACE_EV(ev, it) do { if (blockIdx.x == 5 && blockIdx.y == 7 && (it) < 512) g_trace[ev][it] = clock64(); } while (0)
#else
#define OB_TRACE_EV(ev, it) do { } while (0)
#endif

// ---- the kernel -------------------------------------------------------------------------------

template <int MS, int BN, int NXG, bool AT>
__global__ void __launch_bounds__(Cfg<MS, BN, NXG, AT>::kThreads, 1)
ob_gemm_prefill_kernel(const __grid_constant__ CUtensorMap tmap_b, PrefillArgs a) {
  using C = Cfg<MS, BN, NXG, AT>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  // stage s: [A x MS, 16 KiB each (smem form only)][B BN/64 x 16 KiB][meta x MS, 2 KiB each][bits x MS, 1 KiB each]
  auto stage_a = [&](int s, int t) { return smem_base + s * C::kStageBytes + t * C::kABytes; };
  auto stage_b = [&](int s) { return smem_base + s * C::kStageBytes + MS * C::kABytes; };
  auto stage_e = [&](int s, int t) { return stage_b(s) + C::kBBytes + t * OB_TILE_META_BYTES; };
  auto stage_bits = [&](int s, int t) { return stage_b(s) + C::kBBytes + MS * OB_TILE_META_BYTES + t * OB_TILE_BITS_BYTES; };
  const uint32_t bar_base = smem_base + C::kStages * C::kStageBytes;
  auto bar_full = [&](int s) { return bar_base + 8 * s; };                        // TMA landed
  auto bar_empty = [&](int s) { return bar_base + 8 * (C::kStages + s); };        // MMAs of the stage done
  auto bar_afull = [&](int x) { return bar_base + 8 * (2 * C::kStages + x); };    // +-1 values written to slot x
  auto bar_aempty = [&](int x) { return bar_base + 8 * (2 * C::kStages + C::kASlots + x); };  // MMAs reading slot x done
  const uint32_t bar_acc = bar_base + 8 * (2 * C::kStages + 2 * C::kASlots);
  const uint32_t tmem_slot = bar_acc + 8;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t mb = blockIdx.x;                  // block of MS weight tiles
  const int64_t n0 = (int64_t)blockIdx.y * BN;
  const int kt = (int)(a.k / BK);
  long long budget = 2000000000ll;                // cycles, about a second

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int x = 0; x < C::kASlots; ++x) { mbar_init(bar_afull(x), 128 * MS); mbar_init(bar_aempty(x), 1); }
    mbar_init(bar_acc, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
  }
  if (threadIdx.x == 0) OB_TRACE_EV(7, 2);
  if (warp == 1) tcgen05_alloc(tmem_slot, C::kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;
  const uint32_t tmem_acc = tmem_base;                           // MS accumulators of BN columns
  const uint32_t tmem_e = tmem_base + C::kAccCols;               // metadata slots
  const uint32_t tmem_a = tmem_base + C::kAccCols + C::kECols;   // +-1 operand slots (TMEM form)

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      for (int it = 0; it < kt; ++it) {
        const int s = it % C::kStages;
        mbar_wait(bar_empty(s), ((it / C::kStages) & 1) ^ 1, budget, a.status, 1);
        OB_TRACE_EV(0, it);
        mbar_expect_tx(bar_full(s), C::kTxBytes);
#pragma unroll
        for (int j = 0; j < BN / 64; ++j)
          tma_load_2d(stage_b(s) + j * C::kBBoxBytes, &tmap_b, (int)(n0 + 64 * j), it * BK, bar_full(s));
#pragma unroll
        for (int t = 0; t < MS; ++t) {
          const int64_t tile = (mb * MS + t) * kt + it;
          bulk_load(stage_e(s, t), a.meta_tile + tile * OB_TILE_META_BYTES, OB_TILE_META_BYTES, bar_full(s));
          bulk_load(stage_bits(s, t), a.bits_tile + tile * OB_TILE_BITS_BYTES, OB_TILE_BITS_BYTES, bar_full(s));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 2) /*sparse*/ | (1u << 4) /*fp32 accumulate*/ | (1u << 16) /*B is n-major*/ |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      for (int it = 0; it < kt; ++it) {
        const int s = it % C::kStages, x = it % C::kASlots;
        // "operand full" covers "TMA landed": every expander thread waited for the stage first
        mbar_wait(bar_afull(x), (it / C::kASlots) & 1, budget, a.status, 3);
        OB_TRACE_EV(5, it);
        tcgen05_fence_after();
        const uint64_t bdesc = make_desc(stage_b(s), C::kBBoxBytes, 1024, kLayoutSw128);
#pragma unroll
        for (int t = 0; t < MS; ++t) {
          const uint32_t e_col = tmem_e + 8 * t + 4 * (it & 1);
          tcgen05_cp_128x128b(e_col, make_desc(stage_e(s, t), 128, 128, kLayoutNone));
          const uint64_t adesc = make_desc(stage_a(s, t), 16, 1024, kLayoutSw128);
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            // k-block kb: 32 k-rows (4 KiB) further in B; metadata column kb = even column address + id2;
            // the +-1 operand 32 bytes further along its swizzled smem rows, or 8 TMEM columns further
            if constexpr (AT)
              tcgen05_mma_sp_f16_ts(tmem_acc + t * BN, tmem_a + x * C::kASlotCols + t * 32 + 8 * kb, bdesc + (uint64_t)(256 * kb),
                                    e_col + (kb & ~1), idesc | (uint32_t)(kb & 1), (it | kb) != 0);
            else
              tcgen05_mma_sp_f16(tmem_acc + t * BN, adesc + (uint64_t)(2 * kb), bdesc + (uint64_t)(256 * kb),
                                 e_col + (kb & ~1), idesc | (uint32_t)(kb & 1), (it | kb) != 0);
          }
        }
        tcgen05_commit(bar_empty(s));
        if constexpr (C::kOwnSlotRing) tcgen05_commit(bar_aempty(x));
        OB_TRACE_EV(6, it);
      }
      tcgen05_commit(bar_acc);
    }
  } else if (warp < 2 + 4 * NXG) {
    // ---------------- expander: thread = weight row; the warp's TMEM quadrant is warp % 4 ----------------
    const int xg = (warp - 2) >> 2;                       // expander group
    const int q = warp & 3;
    const int r = q * 32 + lane;
    for (int it = 0; it < kt; ++it) {
      // every group passes every phase of the barriers it ever waits on (parity tracking)
      const int s = it % C::kStages, x = it % C::kASlots;
      mbar_wait(bar_full(s), (it / C::kStages) & 1, budget, a.status, 4);
      if (threadIdx.x == 64) OB_TRACE_EV(1, it);
      if constexpr (C::kOwnSlotRing) mbar_wait(bar_aempty(x), ((it / C::kASlots) & 1) ^ 1, budget, a.status, 6);
      if (threadIdx.x == 64) OB_TRACE_EV(2, it);
#pragma unroll
      for (int t = 0; t < MS; ++t) {
        if ((it * MS + t) % NXG != xg) continue;
        const uint2 w = *reinterpret_cast<const uint2*>(smem_gen + (stage_bits(s, t) - smem_base) + r * 8);
        if constexpr (AT) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 16; ++j) { v[j] = expand_pair(w.x, j); v[16 + j] = expand_pair(w.y, j); }
          tcgen05_fence_after();
          tcgen05_st_32x32b_x32(tmem_a + ((uint32_t)(q * 32) << 16) + (uint32_t)(x * C::kASlotCols + t * 32), v);
          tcgen05_fence_before();
        } else {
          uint8_t* arow = smem_gen + (stage_a(s, t) - smem_base) + r * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint32_t word = (c < 4) ? w.x : w.y;
            uint4 v;
            v.x = expand_pair(word, 4 * (c & 3) + 0);
            v.y = expand_pair(word, 4 * (c & 3) + 1);
            v.z = expand_pair(word, 4 * (c & 3) + 2);
            v.w = expand_pair(word, 4 * (c & 3) + 3);
            *reinterpret_cast<uint4*>(arow + ((c ^ (r & 7)) << 4)) = v;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        mbar_arrive(bar_afull(x));
      }
      if (threadIdx.x == 64) OB_TRACE_EV(3, it);
    }
  } else {
    // ---------------- epilogue: warp quadrant = warp % 4, thread = output row ----------------
    const int q = warp & 3;
    mbar_wait(bar_acc, 0, budget, a.status, 5);
    if (q == 0 && lane == 0) OB_TRACE_EV(7, 0);
    tcgen05_fence_after();
#pragma unroll 1
    for (int t = 0; t < MS; ++t) {
      const int64_t row = (mb * MS + t) * BM + q * 32 + lane;
      const float sc = a.scale ? __half2float(a.scale[row]) : 1.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tcgen05_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(t * BN + c0), v);
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
          for (int j = 0; j < 8; ++j) {
            if (col + 4 * j < a.n) {
              float4 o = make_float4(__uint_as_float(v[4 * j]) * sc, __uint_as_float(v[4 * j + 1]) * sc,
                                     __uint_as_float(v[4 * j + 2]) * sc, __uint_as_float(v[4 * j + 3]) * sc);
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
  if (warp == 1) {
    tcgen05_fence_after();
    tcgen05_dealloc(tmem_base, C::kTmemCols);
  }
  if (threadIdx.x == 0) OB_TRACE_EV(7, 3);
}

// ---- host side ----------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

template <int MS, int BN, int NXG, bool AT>
cudaError_t launch(const CUtensorMap& tmap, const PrefillArgs& a, cudaStream_t stream) {
  using C = Cfg<MS, BN, NXG, AT>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(ob_gemm_prefill_kernel<MS, BN, NXG, AT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  dim3 grid((unsigned)(a.m / (BM * MS)), (unsigned)((a.n + BN - 1) / BN));
  ob_gemm_prefill_kernel<MS, BN, NXG, AT><<<grid, C::kThreads, C::kSmemBytes, stream>>>(tmap, a);
  return cudaGetLastError();
}

}  // namespace

namespace ob {

bool prefill2_supported(int64_t m, int64_t n, int64_t k);
cudaError_t launch_gemm_prefill2(const CUtensorMap* tmap, const CUtensorMap* tmap_c, int ks, bool token_major,
                                 const void* bits_tile, const void* meta_tile, const void* scale, const void* bias,
                                 void* d, int64_t m, int64_t n, int64_t k, int out_type, int* status,
                                 cudaStream_t stream);
int prefill_splitk_choose(int64_t tiles, int64_t kt);
cudaError_t launch_gemm_prefill_splitk(const CUtensorMap* tmap, int S, const void* bits_tile, const void* meta_tile,
                                       const void* scale, void* d, int64_t m, int64_t n, int64_t k, int out_type,
                                       int* status, cudaStream_t stream);
bool prefill3_supported(int64_t m, int64_t n, int64_t k, int out_type, const void* d, bool token_major);
cudaError_t launch_gemm_prefill3(const CUtensorMap* tmap, bool token_major, const void* bits_tile, const void* meta_tile,
                                 const void* scale, const void* bias, void* d, void* const* extra_dst, int n_extra,
                                 int64_t m, int64_t n, int64_t k, int* status, cudaStream_t stream);

namespace {
int forced_variant() {
  static const int forced = [] { const char* v = getenv("ONEBIT_PREFILL_VARIANT"); return v ? atoi(v) : 0; }();
  return forced;
}
}  // namespace

bool prefill_supported(int64_t m, int64_t n, int64_t k) {
  return m % BM == 0 && k % BK == 0 && n % 8 == 0 && n >= 8 && k >= BK;
}

cudaError_t launch_gemm_prefill(const void* bits_tile, const void* meta_tile, const void* scale, const void* b,
                                void* d, int64_t m, int64_t n, int64_t k, int out_type, int* status,
                                cudaStream_t stream) {
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(b) & 15) != 0) return cudaErrorMisalignedAddress;
  // tensor map of B (k x n row-major): boxes of 64 tokens x box_rows k-rows, 128-byte swizzle
  auto make_map = [&](CUtensorMap* tmap, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)k};
    const cuuint64_t strides[1] = {(cuuint64_t)n * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return encode(tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(b), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  };
  // Tuning knob for experiments: ONEBIT_PREFILL_VARIANT = 121 (single CTA, +-1 operand expanded into
  // shared memory: the first version of this kernel, kept as the baseline of the profiling history),
  // 1121 / 1141 / 1221 (single CTA, operand in tensor memory: 128 tokens / 256 tokens / two stacked
  // weight tiles), 2 / 22 (CTA-pair kernel with one / two weight tiles per stage), 3 (persistent CTA-pair
  // kernel), 4 (split-K cluster kernel), 1 (shape heuristic without the CTA-pair kernels).
  const int forced = forced_variant();
  const int64_t row_tiles = m / BM, kt_tiles = k / BK;
  const bool two = (m % 256 == 0);
  const int sms = sm_count();
  // The CTA-pair kernel (256 rows x 256 tokens per pair, each CTA staging half of the token tile) is
  // the fastest once its pairs fill the SM pairs of the chip.
  const bool pair_fits = n > 128 && prefill2_supported(m, n, k) && (row_tiles / 2) * ((n + 255) / 256) >= sms / 2;
  // Its persistent form saves the per-tile start-up (tensor-memory allocation, barrier set-up, first ring
  // of loads) and overlaps the output stores with the next tile: measured +4 % (k = 4096) to +39 %
  // (k = 1024) for short k loops, -1 % to -5 % for k >= 8192, where the stores through TMA win.
  if ((forced == 3 || (forced == 0 && pair_fits && k <= 4096)) && prefill3_supported(m, n, k, out_type, d, false)) {
    CUtensorMap tmap3;
    if (!make_map(&tmap3, BK * 2)) return cudaErrorInvalidValue;
    return launch_gemm_prefill3(&tmap3, false, bits_tile, meta_tile, scale, nullptr, d, nullptr, 0, m, n, k, status, stream);
  }
  if (((forced == 2 || forced == 22) && prefill2_supported(m, n, k)) || (forced == 0 && pair_fits)) {
    const int ks = (forced == 2) ? 1 : 2;
    CUtensorMap tmap2, tmap_c;
    if (!make_map(&tmap2, BK * ks)) return cudaErrorInvalidValue;
    // fp16 C leaves through shared memory and TMA stores: boxes of 64 tokens x 128 rows
    bool c_map = false;
    if (out_type == OB_OUT_F16 && (reinterpret_cast<uintptr_t>(d) & 15) == 0) {
      const cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)m};
      const cuuint64_t strides[1] = {(cuuint64_t)n * 2};
      const cuuint32_t box[2] = {64, (cuuint32_t)BM};
      const cuuint32_t estr[2] = {1, 1};
      c_map = encode(&tmap_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, d, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    return launch_gemm_prefill2(&tmap2, c_map ? &tmap_c : nullptr, ks, false, bits_tile, meta_tile, scale, nullptr, d, m, n,
                                k, out_type, status, stream);
  }
  CUtensorMap tmap;
  if (!make_map(&tmap, BK)) return cudaErrorInvalidValue;
  PrefillArgs a{static_cast<const uint8_t*>(bits_tile), static_cast<const uint8_t*>(meta_tile),
                static_cast<const __half*>(scale), d, m, n, k, out_type, status};
  switch (forced) {
    case 121: return launch<1, 128, 1, false>(tmap, a, stream);
    case 1121: return launch<1, 128, 1, true>(tmap, a, stream);
    case 1141: return launch<1, 256, 1, true>(tmap, a, stream);
    case 1221: if (two) return launch<2, 128, 1, true>(tmap, a, stream); break;
    default: break;
  }
  // Single-CTA variants, all with the +-1 operand in tensor memory: a 256-token tile once it fills
  // the SMs, else two stacked weight tiles sharing 128 tokens, else the smallest tile, which
  // spreads a small problem over the most SMs.
  if (n > 128 && row_tiles * ((n + 255) / 256) >= sms) return launch<1, 256, 1, true>(tmap, a, stream);
  if (two && (row_tiles / 2) * ((n + 127) / 128) >= sms) return launch<2, 128, 1, true>(tmap, a, stream);
  // Too few output tiles to fill the chip: the same 128 x 128 pipeline with k cut over a cluster (variant 4 forces it;
  // with one slice it is the plain single-CTA kernel).
  const int64_t tiles = row_tiles * ((n + 127) / 128);
  const int S = prefill_splitk_choose(tiles, kt_tiles);
  if (forced == 4 || S > 1) return launch_gemm_prefill_splitk(&tmap, S, bits_tile, meta_tile, scale, d, m, n, k, out_type, status, stream);
  return launch<1, 128, 1, true>(tmap, a, stream);
}

// The persistent pair kernel writing the fp16 result to C and to n_extra more buffers of C's shape.
bool prefill_scatter_supported(int64_t m, int64_t n, int64_t k, const void* d) {
  return prefill3_supported(m, n, k, OB_OUT_F16, d, false);
}

cudaError_t launch_gemm_prefill_scatter(const void* bits_tile, const void* meta_tile, const void* scale, const void* b,
                                        void* d, void* const* extra_dst, int n_extra, int64_t m, int64_t n, int64_t k,
                                        int* status, cudaStream_t stream) {
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(b) & 15) != 0) return cudaErrorMisalignedAddress;
  CUtensorMap tmap;
  const cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)k};
  const cuuint64_t strides[1] = {(cuuint64_t)n * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)(2 * BK)};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(b), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  return launch_gemm_prefill3(&tmap, false, bits_tile, meta_tile, scale, nullptr, d, extra_dst, n_extra, m, n, k, status, stream);
}

bool prefill_tokens_supported(int64_t m, int64_t n, int64_t k) { return prefill2_supported(m, 8, k) && n >= 1; }

// Token-major form (the nn.Linear convention): x (n, k) row-major fp16, y (n, m) row-major, optional
// bias (m). Always the CTA-pair kernel: the token tile is a K-major operand loaded straight from x,
// the epilogue writes the transposed tile, so no transposition pass exists anywhere.
cudaError_t launch_gemm_prefill_tokens(const void* bits_tile, const void* meta_tile, const void* scale, const void* bias,
                                       const void* x, void* y, int64_t m, int64_t n, int64_t k, int out_type, int* status,
                                       cudaStream_t stream) {
  EncodeTiledFn encode = get_encode_fn();
  if (!encode) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return cudaErrorMisalignedAddress;
  CUtensorMap tmap_x, tmap_y;
  const cuuint32_t estr[2] = {1, 1};
  {
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)n};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {64, 128};
    if (encode(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  if (forced_variant() == 3 && prefill3_supported(m, n, k, out_type, y, true))
    return launch_gemm_prefill3(&tmap_x, true, bits_tile, meta_tile, scale, bias, y, nullptr, 0, m, n, k, status, stream);
  bool y_map = false;
  if (out_type == OB_OUT_F16 && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
    const cuuint64_t dims[2] = {(cuuint64_t)m, (cuuint64_t)n};
    const cuuint64_t strides[1] = {(cuuint64_t)m * 2};
    const cuuint32_t box[2] = {64, 256};
    y_map = encode(&tmap_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  return launch_gemm_prefill2(&tmap_x, y_map ? &tmap_y : nullptr, 2, true, bits_tile, meta_tile, scale, bias, y, m, n, k,
                              out_type, status, stream);
}

}  // namespace ob

#ifdef OB_TRACE
extern "C" int onebit_debug_read_trace(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_trace, sizeof(long long) * 8 * 512);
}
#endif
