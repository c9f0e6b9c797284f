// K3, tensor-memory form: the few-token kernel (n <= 16 per pass) on the 5th-generation tensor cores.
//
// Same job and same cluster split-K scheme as gemm_decode.cu -- stream the 1.5 bit/weight operand from HBM
// exactly once; a cluster of S CTAs cuts K into S slices; partial sums meet in the row owner's shared memory
// and are added in a fixed order -- but the multiply itself is the tcgen05 pipeline of the large-shape
// kernels, shrunk to a 128 x 16 accumulator:
//   * one CTA = one 128-row block of A x one slice of K. Weights arrive by bulk async copies in rounds of
//     4 tiles (12 KiB) into a shared-memory ring, the whole first ring requested by one thread at kernel
//     start;
//   * 8 worker warps (thread = weight row, two groups of 4 warps taking alternate pairs of tiles) expand a
//     tile's 64 sign bits per row into 32 registers of fp16 +-1 pairs (one integer multiply by a power of two on
//     the FMA pipe + one logic op on the ALU pipe per pair) and store them with tcgen05.st into a ring of
//     tensor-memory slots, one wait and one hand-over per pair; one thread copies the tile's metadata block
//     into tensor memory (tcgen05.cp) and issues 4 x tcgen05.mma.sp.kind::f16 (M = 128, N = 16, K = 32 dense)
//     with the +-1 operand read from tensor memory. The K loop accumulates in tensor memory, so no partial
//     sums of a CTA ever meet in shared memory, no warp reads token fragments, and the legacy mma.sp issue
//     cost (one instruction per 16 x 32 weights and 8 tokens) is gone;
//   * tokens are staged by the worker warps (through registers, or with up to 8 tokens as asynchronous 16-byte
//     copies), each group of 4 warps the tokens of its own pair of tiles, so that the group's one arrival per pair
//     hands over operand slots and tokens together and the MMA warp waits on one barrier per pair and on nothing
//     else (every barrier wait of that warp costs ~100 cycles of its serial instruction stream, which set the
//     CTA's pace). They form the B operand in the canonical no-swizzle layout: core matrices of 8 x 16 bytes.
//     Exception: 16 tokens per pass of B (k, n) under a K split come by TMA, one box of 16 tokens x 128 k rows with
//     the 32-byte swizzle per tile, requested by the weight-stream thread onto the round's weight barrier (see
//     make_token_map for where that pays). Token rows that are contiguous in k (x (n, k), or a single token) become a
//     K-major operand; B (k, n) rows become an N-major operand, 16 bytes = 8 tokens of one k row per piece,
//     so nothing is ever transposed element by element. Token columns beyond n are never written: what
//     the tensor core reads there only reaches accumulator columns that are never stored;
//   * consecutive MMAs go to four separate accumulators (one per 32-k block of a tile): a 128 x 16 MMA is a few
//     cycles of tensor work, and a chain of dependent ones on a single accumulator ran at the pipeline's latency,
//     ~200 cycles each; the four are added in the epilogue in a fixed order;
//   * epilogue: tcgen05.ld (thread = row, 8 token columns per accumulator), then either scale and store (S = 1)
//     or asynchronous 16-byte stores into the owner CTA's shared memory that complete on the owner's mbarrier
//     (st.async): data and signal travel together, so no cluster-wide barrier and no release fence stand between
//     the last MMA and the sum. The owner adds the S slices in a fixed order, scales, stores;
//   * programmatic dependent launch as in gemm_decode.cu. Tensor memory is allocated BEFORE the CTA lets
//     dependents start, and the kernel asks for enough shared memory that at most two CTAs share an SM: a
//     resident CTA of the next grid can then never hold tensor memory that a CTA of this grid still needs.
// Every mbarrier wait is bounded; a wait that gives up records a code in g_fewtok_status, and the kernel still
// runs to its end and frees its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <climits>
#include <cstdlib>

#include "formats.h"
#include "kernels.h"
#include "sm100_ptx.h"

namespace {

using namespace ob_ptx;

// Timeline instrumentation for tuning, compiled in only with -DOB_TRACE: one CTA records the SM clock at the
// hand-overs of its pipeline. Row 0: events of worker thread 0, row 1: events of the MMA thread, rows 2/3: start
// and end of each tile expansion of worker thread 0, rows 4/5: operand ready / MMAs issued per tile (MMA thread),
// rows 6-10: after the metadata copy and after each of the four MMAs.
#ifdef OB_TRACE
__device__ long long g_trace_ft[16][64];
#define OB_TRACE_ON (blockIdx.x == 3 && blockIdx.z == 0 && blockIdx.y == 0)
#define OB_TRACE_EV(ev) do { if (OB_TRACE_ON && (threadIdx.x == 0 || threadIdx.x == 288)) g_trace_ft[threadIdx.x != 0][ev] = clock64(); } while (0)
#define OB_TRACE_TILE(row, t) do { if (OB_TRACE_ON && (t) < 64 && (threadIdx.x == 0 || threadIdx.x == 128 || threadIdx.x == 288)) g_trace_ft[row][t] = clock64(); } while (0)
#define OB_TRACE_ROUND(row, r) do { if (OB_TRACE_ON && (r) < 64 && threadIdx.x == 0) g_trace_ft[row][r] = clock64(); } while (0)
#else
#define OB_TRACE_EV(ev) do { } while (0)
#define OB_TRACE_TILE(row, t) do { } while (0)
#define OB_TRACE_ROUND(row, r) do { } while (0)
#endif

// nonzero once a bounded wait has given up (200 + role code); read and cleared by the host
__device__ int g_fewtok_status;

constexpr int kTileBytes = OB_TILE_META_BYTES + OB_TILE_BITS_BYTES;
constexpr int KL = 4;                    // tiles per round of the weight ring
constexpr int kWorkers = 256;            // warps 0-7: tokens, expansion, epilogue
constexpr int kThreads = kWorkers + 64;  // warp 8: weight stream, warp 9: tensor memory + MMA issue
constexpr int kAccs = 4;                 // independent accumulators of 16 columns (one per 32-k block of a tile)
constexpr int kASlots = 4;               // +-1 operand slots in tensor memory (one tile each); a power of two
constexpr int kTmemCols = 256;           // [0,64) accumulators, [64,80) metadata slots, [96,224) operand slots
constexpr int kTmemE = 64, kTmemA = 96;
constexpr int kPairs = kASlots / 2;      // slots are handed over in pairs of consecutive tiles: one commit per pair
static_assert(kASlots == 4 && KL % 2 == 0, "the slot ring is indexed with masks; a round is whole pairs");
static_assert(kTmemA + 32 * kASlots <= kTmemCols && kTmemE + 4 * kASlots <= kTmemA && 16 * kAccs <= kTmemE, "tensor memory plan");
constexpr int kProdWarp = 8, kMmaWarp = 9;   // weight stream; tensor-memory allocation and MMA issue
constexpr uint32_t kPollNs = 2000;      // a poll of a barrier may sleep this long inside the instruction (it wakes when the phase completes)
constexpr int kMinSmem = 78 * 1024;      // at most two CTAs per SM, whatever the configuration needs

// NG = groups of 8 token columns per pass (the MMA is always N = 16; with NG = 1 both halves read the same tokens)
template <int NG> struct FewTokCfg {
  static constexpr int NP = 8 * NG;
  static constexpr int kRing = (NG == 1) ? 4 : 3;                             // rounds in flight
  static constexpr int kRoundWeights = KL * kTileBytes;                       // [meta of KL tiles | signs of KL tiles]
  static constexpr int kTileTokens = NG * 2048;                               // 128 k x 8 NG tokens, fp16
  static constexpr int kRoundTokens = KL * kTileTokens;
  static constexpr int kWeights = kRing * kRoundWeights;
  static constexpr int kTokens = kRing * kRoundTokens;
  static constexpr int kRecv = 136 * NP * 4;                                  // [source rank][row of this CTA's share][token]; S x ceil(128 / S) <= 133 rows
  static constexpr int kBars = 8 * (2 * kRing + 2 * kPairs + 2) + 8;          // barriers + the tensor-memory address
  static constexpr int kNeeded = kWeights + kTokens + kRecv + kBars + 1024;   // + alignment slack
  static constexpr int kTotal = kNeeded < kMinSmem ? kMinSmem : kNeeded;
  static constexpr int kPieces = KL * 128 * NP / 8 / kWorkers;                // 16-byte token pieces per worker and round
  static_assert(2 * (kTotal + 1024) <= 227 * 1024, "two CTAs per SM must fit");
  static_assert(KL * 128 * NP / 8 == kPieces * kWorkers, "a round's tokens are whole 16-byte pieces per worker");
};

struct FewTokArgs {
  const uint8_t* bits_tile;
  const uint8_t* meta_tile;
  const __half* scale;
  const __half* bias;   // per output row, added after the scale (token-major callers; NULL = none)
  const __half* b;
  void* d;
  int64_t m, n, k;
  int fresh_weights;    // 1: request no weights before the previous kernel of the stream has completed
  int tok_tma;          // 1: B (k, n) with 16 tokens per pass is fetched by TMA (the kernel's tensor-map argument is valid)
  uint32_t pow2[16];    // pow2[p] = 1 << (15 - p): a multiplication by a value the compiler does not know is an integer
                        // multiply-add (FMA pipe), a shift by a constant is an ALU-pipe instruction like the logic
                        // operation that follows it; the expansion is bound by the ALU pipe
};

// start-address field of a shared-memory matrix descriptor: bits 4-17 of the address. The mask matters: inside a
// cluster the shared-window address of a CTA carries its rank in the upper bits
__device__ __forceinline__ uint64_t desc_addr(uint32_t saddr) { return (uint64_t)((saddr >> 4) & 0x3FFFu); }

// true in exactly one lane of a converged warp (the same lane every time)
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

// Four 32-lane x 8-column loads from tensor memory in flight together, one wait for all of them. One asm block: the
// results may not be touched before the wait, and only a data dependency on the block tells the compiler so.
__device__ __forceinline__ void tcgen05_ld_32x32b_x8_four(uint32_t t0, uint32_t t1, uint32_t t2, uint32_t t3, uint32_t (&r)[4][8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%32];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%8, %9, %10, %11, %12, %13, %14, %15}, [%33];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%16, %17, %18, %19, %20, %21, %22, %23}, [%34];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%24, %25, %26, %27, %28, %29, %30, %31}, [%35];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=&r"(r[0][0]), "=&r"(r[0][1]), "=&r"(r[0][2]), "=&r"(r[0][3]), "=&r"(r[0][4]), "=&r"(r[0][5]), "=&r"(r[0][6]), "=&r"(r[0][7]),
        "=&r"(r[1][0]), "=&r"(r[1][1]), "=&r"(r[1][2]), "=&r"(r[1][3]), "=&r"(r[1][4]), "=&r"(r[1][5]), "=&r"(r[1][6]), "=&r"(r[1][7]),
        "=&r"(r[2][0]), "=&r"(r[2][1]), "=&r"(r[2][2]), "=&r"(r[2][3]), "=&r"(r[2][4]), "=&r"(r[2][5]), "=&r"(r[2][6]), "=&r"(r[2][7]),
        "=&r"(r[3][0]), "=&r"(r[3][1]), "=&r"(r[3][2]), "=&r"(r[3][3]), "=&r"(r[3][4]), "=&r"(r[3][5]), "=&r"(r[3][6]), "=&r"(r[3][7])
      : "r"(t0), "r"(t1), "r"(t2), "r"(t3)
      : "memory");
}

// 16 bytes into the shared memory of a CTA of the cluster; the store completes on that CTA's mbarrier (16 bytes of
// its transaction count), so the receiver learns of the data without any further synchronisation
__device__ __forceinline__ void st_async_v4(uint32_t cluster_addr, float x, float y, float z, float w, uint32_t cluster_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(cluster_addr), "f"(x), "f"(y), "f"(z), "f"(w), "r"(cluster_bar) : "memory");
}

// TM = token-major operands (the nn.Linear convention): b is x (n, k) row-major, d is y (n, m) row-major
template <int NG, typename OutT, bool TM>
__global__ void __launch_bounds__(kThreads, 2) ob_gemm_fewtok_kernel(const __grid_constant__ CUtensorMap tok_map, FewTokArgs a) {
  using L = FewTokCfg<NG>;
  constexpr int NP = L::NP, kRing = L::kRing, kPieces = L::kPieces;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

  OB_TRACE_EV(0);
  // the cluster spans the whole y extent of the grid
  const int S = (int)gridDim.y;
  const int rank = (int)blockIdx.y;
  const int64_t mb = blockIdx.x;
  const int64_t n0 = (int64_t)blockIdx.z * NP;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  uint8_t* wring = smem;
  uint8_t* tring = smem + L::kWeights;
  float* s_recv = reinterpret_cast<float*>(smem + L::kWeights + L::kTokens);
  const uint32_t bar0 = smem_base + L::kWeights + L::kTokens + L::kRecv;
  auto bar_wfull = [&](int s) { return bar0 + 8 * s; };                        // a round of weights has landed
  auto bar_wempty = [&](int s) { return bar0 + 8 * (kRing + s); };             // its MMAs are done: weights and tokens free
  auto bar_afull = [&](int y) { return bar0 + 8 * (2 * kRing + y); };          // pair y of a round is ready: both operand slots written and the pair's tokens staged (the 4 warps of group y)
  auto bar_aempty = [&](int y) { return bar0 + 8 * (2 * kRing + kPairs + y); };    // the MMAs reading pair y are done
  const uint32_t bar_acc = bar0 + 8 * (2 * kRing + 2 * kPairs);
  const uint32_t bar_recv = bar_acc + 8;                                       // every slice's sums for this CTA's rows have landed
  const uint32_t tmem_slot = bar_recv + 8;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem + (tmem_slot - smem_base));

  const int tiles_k = (int)(a.k / OB_TILE_K);
  const int tile_begin = (int)((int64_t)tiles_k * rank / S), tile_end = (int)((int64_t)tiles_k * (rank + 1) / S);
  const int T = tile_end - tile_begin;                        // tiles of this CTA's slice
  const int nrounds = (T + KL - 1) / KL;
  long long budget = 2000000000ll;
  const int nvalid = (int)min((int64_t)NP, a.n - n0);

  // token rows contiguous in k (a K-major operand): token-major callers, or a single, 16-byte aligned token
  const bool kmajor = TM || (a.n == 1 && (reinterpret_cast<uintptr_t>(a.b) & 15) == 0);
  const bool vec_rows = !kmajor && (a.n % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.b) & 15) == 0);
  const bool quad_rows = !kmajor && (a.n % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.b) & 7) == 0);
  // whole 16-byte pieces of up to 8 tokens: staged by asynchronous copies (see below). With 16 tokens per pass the
  // register route is faster (measured: 28672 x 8192, 16 tokens: 31 us against 42 us)
  const bool tok_async = NG == 1 && (kmajor || vec_rows);
  // B (k, n) with 16 tokens per pass: a row of the block is 32 bytes, and a TMA box of 16 tokens x 128 k rows with the
  // 32-byte swizzle lands exactly as the tensor core's N-major 32-byte-swizzled operand -- one box per tile on the
  // weight barrier, requested by the weight-stream thread; no worker touches a token
  const bool tok_tma = NG == 2 && !TM && a.tok_tma != 0;

  // split-K hand-off: CTA o of the cluster owns rows [o * rows_per, (o+1) * rows_per) of the block and receives,
  // from every CTA of the cluster (itself included), 16-byte pieces of those rows' sums
  const int rows_per = (128 + S - 1) / S;
  const int rows_owned = max(0, min(rows_per, 128 - rank * rows_per));
  const int npieces = (nvalid + 3) / 4;                       // 16-byte pieces per row and sender
  auto issue = [&](int r) {
    const int s = r % kRing;
    const int nt = min(KL, T - r * KL);
    const int64_t tile = mb * tiles_k + tile_begin + r * KL;
    const uint32_t dst = smem_base + s * L::kRoundWeights;
    mbar_expect_tx(bar_wfull(s), nt * (kTileBytes + (tok_tma ? L::kTileTokens : 0)));
    bulk_load(dst, a.meta_tile + tile * OB_TILE_META_BYTES, nt * OB_TILE_META_BYTES, bar_wfull(s));
    bulk_load(dst + KL * OB_TILE_META_BYTES, a.bits_tile + tile * OB_TILE_BITS_BYTES, nt * OB_TILE_BITS_BYTES, bar_wfull(s));
  };
  // the round's tokens by TMA (the barrier already expects their bytes): x = first token of the block (a multiple of
  // 16 tokens = 32 bytes), y = first k row of the tile
  auto issue_tokens_tma = [&](int r) {
    const int s = r % kRing;
    const int nt = min(KL, T - r * KL);
    for (int j = 0; j < nt; ++j)
      tma_load_2d(smem_base + L::kWeights + s * L::kRoundTokens + j * L::kTileTokens, &tok_map, (int)n0,
                  (tile_begin + r * KL + j) * OB_TILE_K, bar_wfull(s));
  };
  if (warp == kProdWarp) {
    // ---------------- weight stream: round r of the slice -> ring slot r % kRing ----------------
    if (lane == 0) {
      // the barriers of the weight ring first, so that the first ring of loads is out as early as possible
      for (int s = 0; s < kRing; ++s) mbar_init(bar_wfull(s), 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      if (a.fresh_weights) asm volatile("griddepcontrol.wait;" ::: "memory");
      const int npre = min(nrounds, kRing);
      for (int r = 0; r < npre; ++r) issue(r);
      if (tok_tma) {
        // tokens are the previous kernel's results: only after the dependency wait
        if (!a.fresh_weights) asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int r = 0; r < npre; ++r) issue_tokens_tma(r);
      }
      for (int s = 0; s < kRing; ++s) mbar_init(bar_wempty(s), 1);
      for (int y = 0; y < kPairs; ++y) { mbar_init(bar_afull(y), kWorkers / 64); mbar_init(bar_aempty(y), 1); }
      mbar_init(bar_acc, 1);
      mbar_init(bar_recv, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      if (S > 1) mbar_expect_tx(bar_recv, (uint32_t)(S * rows_owned * npieces * 16));
    }
  } else if (warp == kMmaWarp) {
    tcgen05_alloc(tmem_slot, kTmemCols);
    // only now may CTAs of the next grid become resident beside this one
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  OB_TRACE_EV(1);

  // tokens of one round: kPieces 16-byte pieces per worker, fetched into registers, stored as core matrices.
  //   K-major source: piece = 8 k values of token j          -> [tile][j / 8][k chunk][j % 8]
  //   N-major source: piece = 8 tokens (group ng) of k row kk -> [tile][ng][kk]          (16 bytes each)
  // Everything that does not depend on the round is worked out once: the source of the piece in the slice's first
  // round (it then moves on by a fixed stride per round), its place inside a round's staging area, the tile of the
  // round it belongs to (a slice's last round may be short) and whether its tokens exist at all.
  // The tokens of a pair of tiles are staged by the worker group that expands that pair (threads 128 g .. 128 g + 127
  // take tiles 2 g and 2 g + 1 of every round), so that the group's arrival on the pair's "ready" barrier covers them
  // and the MMA warp waits for one barrier per pair and nothing else.
  static_assert(KL == 2 * kPairs && kWorkers == 128 * kPairs, "a group of 128 workers stages the tokens of its two tiles");
  auto piece_index = [&](int i) { return (tid & 127) + 128 * i; };   // among the pieces of this thread's group
  const int tgrp = (tid >> 7) & 1;
  uint32_t tsrc[kPieces];                                     // element offset from a.b (the launcher checks n * k < 2^31)
  uint32_t tplace[kPieces];                                   // bits 0-23: byte offset in the staging area, 24-31: tile
#pragma unroll
  for (int i = 0; i < kPieces; ++i) {
    const int idx = piece_index(i);
    if (kmajor) {
      const int j = idx % NP, c = 32 * tgrp + idx / NP;       // token, 8-k chunk of the round (16 chunks per tile)
      const int tile = (j < nvalid) ? (c >> 4) : KL;          // KL = never
      tsrc[i] = (uint32_t)((n0 + j) * a.k + (int64_t)tile_begin * OB_TILE_K + c * 8);
      tplace[i] = (uint32_t)((c >> 4) * L::kTileTokens + (j >> 3) * 2048 + (c & 15) * 128 + (j & 7) * 16) | ((uint32_t)tile << 24);
    } else {
      const int kk = 256 * tgrp + idx / NG, ng = idx % NG;    // k row of the round, token group
      const int tile = (8 * ng < nvalid) ? (kk >> 7) : KL;
      tsrc[i] = (uint32_t)(((int64_t)tile_begin * OB_TILE_K + kk) * a.n + n0 + 8 * ng);
      tplace[i] = (uint32_t)((kk >> 7) * L::kTileTokens + ng * 2048 + (kk & 127) * 16) | ((uint32_t)tile << 24);
    }
  }
  const uint32_t tstride = (uint32_t)(KL * OB_TILE_K * (kmajor ? 1 : a.n));   // elements from one round to the next
  auto fetch_tokens = [&](int r, uint4 (&tv)[kPieces]) {
    const int ntile = min(KL, T - r * KL);
#pragma unroll
    for (int i = 0; i < kPieces; ++i) {
      tv[i] = make_uint4(0, 0, 0, 0);
      if ((int)(tplace[i] >> 24) < ntile) {
        const __half* src = a.b + tsrc[i];
        if (kmajor || vec_rows) {
          tv[i] = __ldg(reinterpret_cast<const uint4*>(src));
        } else if (quad_rows) {
          const int ng = piece_index(i) % NG;
          uint2* h4 = reinterpret_cast<uint2*>(&tv[i]);       // n % 4 == 0: whole groups of four tokens
          h4[0] = __ldg(reinterpret_cast<const uint2*>(src));
          if (8 * ng + 4 < nvalid) h4[1] = __ldg(reinterpret_cast<const uint2*>(src + 4));
        } else {
          const int ng = piece_index(i) % NG;
          __half* h = reinterpret_cast<__half*>(&tv[i]);
#pragma unroll
          for (int jj = 0; jj < 8; ++jj)
            if (8 * ng + jj < nvalid) h[jj] = src[jj];
        }
      }
      tsrc[i] += tstride;
    }
  };
  auto store_tokens = [&](int r, const uint4 (&tv)[kPieces]) {
    const int ntile = min(KL, T - r * KL);
    uint8_t* sb = tring + (r % kRing) * L::kRoundTokens;
#pragma unroll
    for (int i = 0; i < kPieces; ++i)
      if ((int)(tplace[i] >> 24) < ntile) *reinterpret_cast<uint4*>(sb + (tplace[i] & 0xFFFFFFu)) = tv[i];
  };

  // Whole 16-byte pieces (token rows contiguous in k, or B (k, n) with n % 8 == 0) do not pass through registers at
  // all: every worker issues its pieces of a round as asynchronous 16-byte copies (cp.async) at the top of the round and
  // waits for them only after it has expanded its pair of tiles, right before it arrives on the pair's barrier (by then
  // they have long landed). Other alignments and token counts keep the register route.
  auto issue_tokens_async = [&](int r) {
    const int ntile = min(KL, T - r * KL);
    const uint32_t sb = smem_base + L::kWeights + (r % kRing) * L::kRoundTokens;
#pragma unroll
    for (int i = 0; i < kPieces; ++i) {
      if ((int)(tplace[i] >> 24) < ntile)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sb + (tplace[i] & 0xFFFFFFu)), "l"(a.b + tsrc[i]) : "memory");
      tsrc[i] += tstride;
    }
  };
  uint4 tv[kPieces];
  if (warp < 8) {
    asm volatile("griddepcontrol.wait;" ::: "memory");        // the previous kernel's results (the tokens) are complete
    if (!tok_async && !tok_tma) fetch_tokens(0, tv);
  }
  tcgen05_fence_before();
  __syncthreads();                                            // the barriers exist, the tensor-memory address is written
  tcgen05_fence_after();
  // Every CTA of the cluster announces that it runs; the matching wait stands right before the first store into
  // another CTA's shared memory, which must not be touched before that CTA has started.
  if (S > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_gen;
  OB_TRACE_EV(2);

#define WORKER_WAIT(bar, par, code) mbar_wait_sleepy(bar, par, kPollNs, budget, &g_fewtok_status, code)
  if (warp < 8) {
    // ---------------- workers: stage tokens, expand sign bits into tensor memory ----------------
    // Group g (warps 4g .. 4g+3, one 32-row quadrant each) owns pair g of every round: tiles 2g and 2g + 1 and the
    // operand slots of the same numbers. A warp expands both tiles of its pair back to back, waits once for the two
    // tensor-memory stores and arrives once; the other group works on the other pair at the same time.
    const int q = warp & 3, grp = warp >> 2;
    const int row = q * 32 + lane;
    const uint32_t a_col = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(kTmemA + 64 * grp);
    // one word of 32 sign bits -> 16 registers of two fp16 +-1 each: bit p to bit 15, bit p + 16 to bit 31
    // one tile row = two words of 32 sign bits -> 32 registers of two fp16 +-1 each: bit p of a word to bit 15, bit
    // p + 16 to bit 31 of its register p. All multiplies first, then all logic operations: left to itself the compiler
    // paired each multiply with its dependent logic operation and the chain ran at the instructions' latency.
    auto expand_tile = [&](uint2 w, uint32_t (&v)[32]) {
#pragma unroll
      for (int p = 0; p < 15; ++p) { v[p] = w.x * a.pow2[p]; v[16 + p] = w.y * a.pow2[p]; }
      v[15] = w.x;
      v[31] = w.y;
#pragma unroll
      for (int p = 0; p < 32; ++p) asm volatile("lop3.b32 %0, %0, 0x80008000, 0xBC00BC00, 0x6A;" : "+r"(v[p]));   // (v & mask) ^ (-1.0h, -1.0h)
    };
    int s = 0;
#pragma unroll 1
    for (int r = 0; r < nrounds; ++r) {
      OB_TRACE_ROUND(12, r);
      // The token slot of this round was last read by this group's pair of round r - kRing. No wait for it: in round
      // r - 1 this warp has seen the commit that followed its pair of round r - 2 (the wait before the tensor-memory
      // stores below), and a commit completes only after every MMA issued before it, those of round r - kRing
      // (kRing >= 3) among them.
      static_assert(kRing >= 3, "the pair barrier seen a round ago must cover the round that used the token slot");
      if (tok_async) {
        // the tokens of this group's pair set off now; they are needed only when the pair is handed to the MMA warp
        issue_tokens_async(r);
      } else if (!tok_tma) {
        OB_TRACE_ROUND(13, r);
        store_tokens(r, tv);                                  // handed over with the pair (proxy fence and arrival below)
        OB_TRACE_ROUND(14, r);
        if (r + 1 < nrounds) fetch_tokens(r + 1, tv);         // in flight while this round is expanded
      }
      WORKER_WAIT(bar_wfull(s), (r / kRing) & 1, 202);
      OB_TRACE_ROUND(15, r);
      if (r == 0) OB_TRACE_EV(3);
      const int nt = min(KL, T - r * KL);
      if (2 * grp < nt) {
        const uint8_t* sw = wring + s * L::kRoundWeights + KL * OB_TILE_META_BYTES + 2 * grp * OB_TILE_BITS_BYTES + row * 8;
        const bool two = 2 * grp + 1 < nt;                    // an odd slice ends with half a pair
        const uint2 w0 = *reinterpret_cast<const uint2*>(sw);
        uint2 w1 = make_uint2(0, 0);
        if (two) w1 = *reinterpret_cast<const uint2*>(sw + OB_TILE_BITS_BYTES);
        OB_TRACE_TILE(2, r * KL + 2 * grp);
        uint32_t v[32];
        expand_tile(w0, v);                                   // before the wait: only the store needs the slot
        WORKER_WAIT(bar_aempty(grp), (r & 1) ^ 1, 203);       // the MMAs that read this pair of slots a round ago are done
        __syncwarp();        // the tcgen05 instructions below are .sync.aligned: no lane may still be in the wait loop
        tcgen05_fence_after();
        tcgen05_st_32x32b_x32_nowait(a_col, v);
        if (two) {
          expand_tile(w1, v);
          tcgen05_st_32x32b_x32_nowait(a_col + 32, v);
        }
        tcgen05_wait_st();
        tcgen05_fence_before();
        // the pair's tokens: this thread's copies have landed (or were stored at the top of the round); the tensor
        // core reads them through the async proxy
        if (tok_async) asm volatile("cp.async.wait_all;" ::: "memory");
        fence_proxy_async();
        OB_TRACE_TILE(3, r * KL + 2 * grp);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_afull(grp));
      }
      if (++s == kRing) s = 0;
    }
    OB_TRACE_EV(4);
  } else if (warp == kProdWarp) {
    // ---------------- weight stream: refill a slot once its round has been multiplied ----------------
    if (lane == 0) {
      for (int r = kRing; r < nrounds; ++r) {
        mbar_wait_sleepy(bar_wempty(r % kRing), ((r / kRing) - 1) & 1, kPollNs, budget, &g_fewtok_status, 204);
        issue(r);
        if (tok_tma) issue_tokens_tma(r);
      }
    }
  } else {
    // ---------------- MMA issuer ----------------
    // M = 128, N = 16, sparse, fp32 accumulate; B is K-major (bit 16 clear) or N-major (bit 16 set)
    const uint32_t idesc = (1u << 2) | (1u << 4) | (kmajor ? 0u : (1u << 16)) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    // no-swizzle core matrices: 128 bytes between 8-k groups (leading offset), 2048 between the two token groups
    // (stride offset; 0 with one group: both halves of the 16 columns then read the same tokens)
    // TMA-staged tokens: one 32-byte-swizzled atom of 16 tokens x 8 k rows every 256 bytes (stride offset), a single
    // atom along the tokens (leading offset unused), 1024 bytes per 32-k block
    const uint64_t tok_desc = tok_tma ? make_desc(0, 4096, 256, kLayoutSw32) : make_desc(0, 128, (NG == 2) ? 2048u : 0u, kLayoutNone);
    const uint32_t tok_kb = tok_tma ? 64u : 32u;             // descriptor address units (16 bytes) per 32-k block
    const uint64_t meta_desc = make_desc(0, 128, 128, kLayoutNone);
    // The whole warp walks the loop, converged: all lanes wait on the barriers and work out the same descriptors and
    // tensor-memory addresses, which the compiler can therefore keep as warp-uniform values; only the tcgen05
    // instructions themselves are predicated on one elected lane. With the elected lane running the loop alone every
    // operand had to be moved to the uniform datapath per instruction (30-45 cycles per tcgen05 instruction;
    // 25600^2, n = 1: 50.9 us against 47.6 us this way); issued from a branch on the lane number it was 60-75.
    const bool leader = elect_one();
    {
      static_assert(KL == 4 && kPairs == 2 && kASlots == 4, "pair pp of a round is barrier pair pp and operand slots 2 pp, 2 pp + 1");
      int s = 0;                                              // ring slot of the round
      // Whether the next pair is ready is asked BEFORE the commit of the pair in hand: the answer travels while the
      // commit is issued, and the workers are normally ahead, so that the warp rarely stands at a barrier at all.
      bool ready = false;
#pragma unroll 1
      for (int r = 0; r < nrounds; ++r) {
        const int nt = min(KL, T - r * KL);
        // No wait for the round's weights or tokens here: a pair's barrier completes only after its four worker warps
        // have seen the weights land (they read the sign bits) and have staged and fenced the pair's tokens.
#pragma unroll
        for (int pp = 0; pp < KL / 2; ++pp) {
          if (2 * pp < nt) {
            OB_TRACE_TILE(11, r * KL + 2 * pp);
            if (!ready) mbar_wait_sleepy(bar_afull(pp), r & 1, kPollNs, budget, &g_fewtok_status, 207);
            OB_TRACE_TILE(4, r * KL + 2 * pp);
            tcgen05_fence_after();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int j = 2 * pp + h;
              if (j < nt) {
                const int t = r * KL + j;
                const uint32_t e_col = tmem_base + kTmemE + 4 * j;
                if (leader) tcgen05_cp_128x128b(e_col, meta_desc | desc_addr(smem_base + s * L::kRoundWeights + j * OB_TILE_META_BYTES));
                OB_TRACE_TILE(6, t);
                const uint64_t tok = tok_desc | desc_addr(smem_base + L::kWeights + s * L::kRoundTokens + j * L::kTileTokens);
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) {
                  if (leader) tcgen05_mma_sp_f16_ts(tmem_base + 16 * kb, tmem_base + kTmemA + 32 * j + 8 * kb, tok + (uint64_t)(tok_kb * kb),
                                                    e_col + (kb & ~1), idesc | (uint32_t)(kb & 1), t != 0);
                  OB_TRACE_TILE(7 + kb, t);
                }
              }
            }
            // the pair that follows: pair 1 of this round, or pair 0 of the next one
            ready = false;
            if (pp == 0) { if (2 < nt) ready = mbar_try_wait(bar_afull(1), r & 1); }
            else if (r + 1 < nrounds) ready = mbar_try_wait(bar_afull(0), (r + 1) & 1);
            if (leader) tcgen05_commit(bar_aempty(pp));
            OB_TRACE_TILE(5, r * KL + 2 * pp);
          }
        }
        if (leader) tcgen05_commit(bar_wempty(s));             // the round's weights and tokens are free again
        if (++s == kRing) s = 0;
      }
      if (leader) tcgen05_commit(bar_acc);
    }
  }
  __syncwarp();

  // ---------------- epilogue ----------------
  auto finish = [&](int64_t row, int j, float sum, float scale, float bias) {
    sum = __fmul_rn(sum, scale);                              // two roundings, like the other kernels' epilogues
    if (a.bias) sum = __fadd_rn(sum, bias);
    if (j < nvalid) {
      const int64_t o = TM ? (n0 + j) * a.m + row : row * a.n + n0 + j;
      if constexpr (sizeof(OutT) == 2) static_cast<__half*>(a.d)[o] = __float2half_rn(sum);
      else static_cast<float*>(a.d)[o] = sum;
    }
  };
  if (warp < 8) {
    const int q = warp & 3, grp = warp >> 2;
    if (grp < NG) {
      const int row = q * 32 + lane;
      // the per-row constants of an unsplit block: on their way while the last MMAs complete
      const int64_t grow = mb * 128 + row;
      float scale = 1.f, bias = 0.f;
      if (S == 1) {
        if (a.scale) scale = __half2float(a.scale[grow]);
        if (a.bias) bias = __half2float(a.bias[grow]);
      }
      mbar_wait(bar_acc, 0, budget, &g_fewtok_status, 208);
      __syncwarp();          // .sync.aligned loads follow
      tcgen05_fence_after();
      // the four accumulators, added in a fixed order
      float v[8];
      {
        static_assert(kAccs == 4, "the epilogue reads four accumulators");
        uint32_t u[kAccs][8];
        const uint32_t acc0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(8 * grp);
        tcgen05_ld_32x32b_x8_four(acc0, acc0 + 16, acc0 + 32, acc0 + 48, u);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[j] = (__uint_as_float(u[0][j]) + __uint_as_float(u[1][j])) + (__uint_as_float(u[2][j]) + __uint_as_float(u[3][j]));
      }
      tcgen05_fence_before();
      OB_TRACE_EV(5);
      if (S == 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) finish(grow, 8 * grp + j, v[j], scale, bias);
      } else {
        // all CTAs of the cluster have started and initialised their barriers (see the arrive above)
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
        const uint32_t owner = (uint32_t)(row / rows_per);
        const uint32_t local = smem_base + L::kWeights + L::kTokens + (uint32_t)(((rank * rows_per + row % rows_per) * NP + 8 * grp) * 4);
        const uint32_t dst = map_to_cta(local, owner), dbar = map_to_cta(bar_recv, owner);
        if (8 * grp < nvalid) st_async_v4(dst, v[0], v[1], v[2], v[3], dbar);
        if (8 * grp + 4 < nvalid) st_async_v4(dst + 16, v[4], v[5], v[6], v[7], dbar);
      }
    } else if (S > 1) {
      asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    }
  } else if (S > 1) {
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
  }
  if (S > 1) {
    // the per-row constants of this thread's outputs, fetched while the sums travel
    constexpr int kOut = (128 * NP / 2 + kThreads - 1) / kThreads;   // outputs per thread at S = 2, the most
    float sc[kOut], bs[kOut];
#pragma unroll
    for (int i = 0; i < kOut; ++i) {
      const int e = tid + i * kThreads;
      sc[i] = 1.f; bs[i] = 0.f;
      if (e < rows_owned * NP) {
        const int rr = TM ? e % rows_owned : e / NP;
        const int64_t row = mb * 128 + rank * rows_per + rr;
        if (a.scale) sc[i] = __half2float(a.scale[row]);
        if (a.bias) bs[i] = __half2float(a.bias[row]);
      }
    }
    mbar_wait(bar_recv, 0, budget, &g_fewtok_status, 209);    // every slice's sums for this CTA's rows have landed
    OB_TRACE_EV(6);
    // fixed-order sum of the S slices from this CTA's own shared memory
#pragma unroll
    for (int i = 0; i < kOut; ++i) {
      const int e = tid + i * kThreads;
      if (e < rows_owned * NP) {
        // consecutive threads walk the fastest output dimension: tokens of a row (m x n), rows of a token (n x m)
        const int rr = TM ? e % rows_owned : e / NP, j = TM ? e / rows_owned : e % NP;
        if (j < nvalid) {
          float sum = 0.f;
          for (int sl = 0; sl < S; ++sl) sum += s_recv[(sl * rows_per + rr) * NP + j];
          finish(mb * 128 + rank * rows_per + rr, j, sum, sc[i], bs[i]);
        }
      }
    }
  }
  OB_TRACE_EV(7);
  tcgen05_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tcgen05_fence_after();
    tcgen05_dealloc(tmem_base, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Tensor map of B (k, n) row-major for the 16-token passes: boxes of 16 tokens x 128 k rows, 32-byte swizzle, zero
// fill beyond n. False if this B cannot be described or the route is not taken (then the workers stage the tokens).
// Measured (us per call, workers / TMA): 25600^2 in 4 slices 55.0 / 47.8, 11008 x 4096 in 3 slices 7.7 / 7.5,
// 4096 x 11008 in 8 slices 7.8 / 7.7, but 28672 x 8192 unsplit 23.2 / 26.8 (every CTA asks L2 for the same token rows
// at the same time, 32 bytes per request, and TMA does not go through the L1 the two CTAs of an SM share) and
// 4096^2 in 8 slices of 4 tiles 5.6 / 5.8 (a slice of one round: 256 threads fetch it faster than one box per tile).
// Hence: only with a K split and slices of at least two rounds. ONEBIT_FEWTOK_TMA = 0 / 1 forces it off / on.
bool make_token_map(CUtensorMap* map, const void* b, int64_t n, int64_t k, int S) {
  static const int forced = [] { const char* v = getenv("ONEBIT_FEWTOK_TMA"); return v ? (atoi(v) != 0 ? 1 : 0) : -1; }();
  EncodeTiledFn encode = encode_tiled_fn();
  if (forced == 0 || !encode || n % 8 != 0 || (reinterpret_cast<uintptr_t>(b) & 15) != 0) return false;
  if (forced != 1 && (S < 2 || k / OB_TILE_K / S < 2 * KL)) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)k};
  const cuuint64_t strides[1] = {(cuuint64_t)n * 2};
  const cuuint32_t box[2] = {16, (cuuint32_t)OB_TILE_K};
  const cuuint32_t estr[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(b), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NG, typename OutT, bool TM>
cudaError_t launch(const FewTokArgs& a_in, int S, cudaStream_t stream) {
  using L = FewTokCfg<NG>;
  FewTokArgs a = a_in;
  CUtensorMap tok_map = {};
  a.tok_tma = (NG == 2 && !TM && make_token_map(&tok_map, a.b, a.n, a.k, S)) ? 1 : 0;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(ob_gemm_fewtok_kernel<NG, OutT, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(a.m / 128), (unsigned)S, (unsigned)((a.n + L::NP - 1) / L::NP));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)S;
  attr[0].val.clusterDim.z = 1;
  // let this grid start while the previous kernel of the stream drains (ONEBIT_PDL=0 turns it off)
  static const bool pdl = [] { const char* v = getenv("ONEBIT_PDL"); return !(v && atoi(v) == 0); }();
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, ob_gemm_fewtok_kernel<NG, OutT, TM>, tok_map, a);
}

// K split over a cluster of S CTAs (1..8; the slices need not be equal). Two CTAs share an SM, so a wave holds
// 2 x SMs CTAs; a CTA costs a fixed start-up (allocation, barriers, one DRAM round trip) plus its tiles, and a
// split costs the hand-off of the partial sums. S minimises waves x (start-up + tiles) + hand-off in that model,
// whose constants are cycles measured with the kernel's own timeline.
int pick_split(int64_t m, int64_t k, int64_t token_blocks) {
  const int64_t tiles_k = k / OB_TILE_K, row_blocks = m / 128;
  const long long wave = 2ll * ob::sm_count();
  constexpr long long kStart = 2500, kTile = 270, kHandOff = 800;
  int best = 1;
  long long best_cost = LLONG_MAX;
  for (int S = 1; S <= 8; ++S) {
    if (tiles_k < S) break;
    // every block of 16 token columns is a grid of its own along z and streams the weights again (from L2)
    const long long ctas = row_blocks * S * token_blocks, waves = (ctas + wave - 1) / wave, T = (tiles_k + S - 1) / S;
    const long long cost = waves * (kStart + T * kTile) + (S > 1 ? kHandOff : 0);
    if (cost < best_cost) { best = S; best_cost = cost; }
  }
  static const int forced = [] { const char* v = getenv("ONEBIT_DECODE_SPLIT"); return v ? atoi(v) : 0; }();
  if (forced >= 1 && forced <= 8 && forced <= tiles_k) best = forced;
  return best;
}

template <bool TM>
cudaError_t dispatch(const FewTokArgs& a, int out_type, cudaStream_t stream) {
  const bool two = (a.n > 8);
  const int S = pick_split(a.m, a.k, two ? (a.n + 15) / 16 : 1);
  if (out_type == OB_OUT_F16) return two ? launch<2, __half, TM>(a, S, stream) : launch<1, __half, TM>(a, S, stream);
  return two ? launch<2, float, TM>(a, S, stream) : launch<1, float, TM>(a, S, stream);
}

}  // namespace

namespace ob {

cudaError_t launch_gemm_fewtok(const void* bits_tile, const void* meta_tile, const void* scale, const void* bias,
                               const void* b, void* d, int64_t m, int64_t n, int64_t k, int out_type, bool token_major,
                               bool fresh_weights, cudaStream_t stream) {
  FewTokArgs a{static_cast<const uint8_t*>(bits_tile), static_cast<const uint8_t*>(meta_tile),
               static_cast<const __half*>(scale), static_cast<const __half*>(bias), static_cast<const __half*>(b), d, m, n, k,
               fresh_weights ? 1 : 0, 0, {}};
  for (int p = 0; p < 16; ++p) a.pow2[p] = 1u << (15 - p);
  if (k * (n > 1 ? n : 1) >= (int64_t)1 << 31) return cudaErrorInvalidValue;   // token offsets are 32-bit in the kernel
  return token_major ? dispatch<true>(a, out_type, stream) : dispatch<false>(a, out_type, stream);
}

// Reads and clears this kernel's wait status on the current device (0 = no wait gave up).
cudaError_t read_fewtok_status(int* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_fewtok_status, sizeof(int));
  if (e != cudaSuccess || *out == 0) return e;
  const int zero = 0;
  return cudaMemcpyToSymbol(g_fewtok_status, &zero, sizeof(int));
}

}  // namespace ob

#ifdef OB_TRACE
extern "C" int onebit_debug_read_trace_fewtok(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_trace_ft, sizeof(long long) * 16 * 64);
}
#endif
