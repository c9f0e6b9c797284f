// K3: the decode-regime kernel (few tokens, n <= 16 per pass): streams the 1.5 bit/weight operand
// from HBM exactly once and is meant to be bound by that stream, not by arithmetic.
//
// Replaces the reference's 128x64x128 CUTLASS threadblock (csrc/kernel.h:23-25) for the shapes
// where its 64-wide token tile is almost empty. Such a call moves only a few MiB, so the kernel is
// built to be short: the whole grid is one wave, every weight byte of a CTA is requested in the
// first few hundred cycles, and no cluster-wide barrier stands between its last MMA and its result.
//   * one CTA = one 128-row block of A x one slice of K (a cluster of S CTAs cuts K into S slices);
//   * weights: the tile order keeps the metadata (2 KiB) and sign (1 KiB) blocks of consecutive
//     k tiles of a row block adjacent, so a round of KL tiles is two bulk async copies into a
//     shared-memory ring. One thread issues the first ring right after initialising the mbarriers
//     -- 36-48 KiB per CTA in flight before anything else happens -- and refills a slot once all
//     8 warps have read it (longer slices only);
//   * 8 warps = 2 row sets x 4 tile lanes: a warp multiplies four 16-row groups (64 rows) by ONE tile
//     of the round, so that a token fragment read from shared memory feeds four tensor-core
//     instructions; with one row group per warp the kernel was bound by the shared-memory port, not
//     by HBM;
//   * the 2:4 gather is done by the tensor core: sign words are expanded in registers to fp16 +-1
//     pairs (one shift + one logic op per pair, see the tile order in formats.h) and fed with the
//     metadata words to mma.sp m16n8k32 with fp32 accumulation;
//   * tokens (B, k x n row-major, or x, n x k row-major) are staged TRANSPOSED in shared memory (one
//     padded row per token and tile; columns beyond n read one shared row of zeros), so that a B
//     fragment register is one 32-bit load; the global loads of all rounds in the ring are issued together;
//   * reduction: the KL partial sums of a CTA are added through shared memory (the drained weight
//     ring); with S > 1 every thread then PUSHES 16 bytes of sums through distributed shared memory into
//     the CTA that owns those output rows (remote stores are slow to issue: one per thread). The store is an
//     st.async that completes on the owner's mbarrier, so data and signal travel together; each CTA waits for its
//     own barrier only, then adds the S slices in a fixed order, scales, converts and stores. No atomics, no
//     scratch in HBM, no remote reads, no cluster barrier after start-up, deterministic;
//   * programmatic dependent launch: the grid may start while the previous kernel of the stream
//     drains. Packed weights are long-lived, so their loads go out first; the tokens are read, and
//     global memory is written, only after griddepcontrol.wait.
// Every mbarrier wait is bounded; a wait that gives up records a code in g_decode_status.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <climits>
#include <cstdlib>

#include "formats.h"
#include "kernels.h"
#include "sm100_ptx.h"


namespace {

using ob_ptx::expand_pair;

// Timeline instrumentation for tuning, compiled in only with -DOB_TRACE.
#ifdef OB_TRACE
__device__ long long g_trace_dec[4][16];
#define OB_TRACE_EV(ev) do { if (blockIdx.x == 3 && blockIdx.z == 0 && (threadIdx.x == 0 || threadIdx.x == blockDim.x - 1) && blockIdx.y < 2) g_trace_dec[blockIdx.y * 2 + (threadIdx.x != 0)][ev] = clock64(); } while (0)
#else
#define OB_TRACE_EV(ev) do { } while (0)
#endif

// nonzero once a bounded wait has given up (100 + role code); read and cleared by the host
__device__ int g_decode_status;

constexpr int kTileBytes = OB_TILE_META_BYTES + OB_TILE_BITS_BYTES;
constexpr int kTokStride = OB_TILE_K + 8;            // halves per token row of one tile; +8 skews the rows over the banks

// geometry and dynamic shared memory of one CTA; two CTAs share an SM
template <int NT> struct DecodeCfg {
  static constexpr int NP = NT * 8;                                           // token columns per pass
  // 8 warps; two CTAs share an SM, which leaves each thread 128 registers. (16 warps of 64 registers
  // were slower: the sign expansion is integer-ALU work that more warps do not speed up, and they spill.)
  static constexpr int kThreads = 256;
  static constexpr int RG = 4;                                                // 16-row groups per warp (64 rows)
  static constexpr int RS = 8 / RG;                                           // row sets per CTA
  static constexpr int KL = (kThreads / 32) / RS;                             // tile lanes = tiles per round
  static constexpr int kRing = (NT == 1) ? 4 : 3;                             // rounds in flight
  static constexpr int kPieces = KL * OB_TILE_K * NP / 8 / kThreads;          // 16-byte token pieces per thread and round
  static constexpr int kRoundWeights = KL * kTileBytes;                       // [meta of KL tiles | signs of KL tiles]
  static constexpr int kTileTokens = NP * kTokStride * 2;                     // one tile's tokens, transposed
  static constexpr int kRoundTokens = KL * kTileTokens;
  static constexpr int kWeights = kRing * kRoundWeights;
  static constexpr int kTokens = kRing * kRoundTokens;
  static constexpr int kRecv = 128 * NP * 4;                                  // [source rank][row of this CTA's share][token]
  static constexpr int kRed = KL * 128 * NP * 4;                              // [tile lane][row][token], reuses the drained ring
  static_assert(kRed <= kWeights + kTokens, "the reduction buffer must fit the drained ring");
  static constexpr int kBars = (2 * kRing + 2) * 8;                           // [full | empty][slot], the receive barrier, 8 bytes of padding: what follows is accessed 16 bytes at a time
  static constexpr int kZeroRow = (kTokStride * 2 + 15) / 16 * 16;            // a token row of zeros
  static_assert(kBars % 16 == 0 && kRecv % 16 == 0 && (kWeights + kTokens) % 16 == 0, "the zero row behind the barriers is written with 16-byte stores");
  static constexpr int kTotal = kWeights + kTokens + kRecv + kBars + kZeroRow;
  static_assert(2 * (kTotal + 1024) <= 227 * 1024, "two CTAs per SM must fit");
  static_assert(KL * OB_TILE_K * NP / 8 == kPieces * kThreads, "a round's tokens are whole 16-byte pieces per thread");
};

__device__ __forceinline__ void mma_sp_16832(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[4],
                                             uint32_t e) {
  asm volatile(
      "mma.sp::ordered_metadata.sync.aligned.m16n8k32.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, "
      "{%4,%5,%6,%7}, {%8,%9,%10,%11}, {%0,%1,%2,%3}, %12, 0x0;\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(e));
}

struct DecodeArgs {
  const uint8_t* bits_tile;
  const uint8_t* meta_tile;
  const __half* scale;
  const __half* bias;   // per output row, added after the scale (token-major callers; NULL = none)
  const __half* b;
  void* d;
  int64_t m, n, k;
  int fresh_weights;    // 1: the weight buffers were written by the kernel launched just before this one
};

// NT = number of 8-token tiles per pass (1 or 2)
// TM = token-major operands (the nn.Linear convention): b is x (n, k) row-major, d is y (n, m) row-major
template <int NT, typename OutT, bool TM>
__global__ void __launch_bounds__(DecodeCfg<NT>::kThreads, 2) ob_gemm_decode_kernel(DecodeArgs a) {
  using L = DecodeCfg<NT>;
  constexpr int NP = L::NP, RG = L::RG, RS = L::RS, KL = L::KL, kRing = L::kRing, kPieces = L::kPieces, kThreads = L::kThreads;
  extern __shared__ __align__(128) uint8_t smem[];

  OB_TRACE_EV(0);
  // the cluster spans the whole y extent of the grid: rank and size come from the launch geometry,
  // which is cheaper to read at kernel start than the cluster special registers
  const int S = (int)gridDim.y;
  const int rank = (int)blockIdx.y;
  const int64_t mb = blockIdx.x;
  const int64_t n0 = (int64_t)blockIdx.z * NP;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rs = warp % RS, kl = warp / RS;                   // row set, tile lane
  const int g = lane >> 2, t = lane & 3;

  uint8_t* wring = smem;
  __half* stok = reinterpret_cast<__half*>(smem + L::kWeights);
  float* s_recv = reinterpret_cast<float*>(smem + L::kWeights + L::kTokens);
  const uint32_t bar0 = ob_ptx::smem_u32(smem + L::kWeights + L::kTokens + L::kRecv);
  const __half* zrow = reinterpret_cast<const __half*>(smem + L::kWeights + L::kTokens + L::kRecv + L::kBars);
  if (tid < L::kZeroRow / 16) reinterpret_cast<uint4*>(smem + L::kWeights + L::kTokens + L::kRecv + L::kBars)[tid] = make_uint4(0, 0, 0, 0);
  auto bar_full = [&](int s) { return bar0 + 8 * s; };
  auto bar_empty = [&](int s) { return bar0 + 8 * (kRing + s); };
  const uint32_t bar_recv = bar0 + 8 * (2 * kRing);           // every slice's sums for this CTA's rows have landed

  const int tiles_k = (int)(a.k / OB_TILE_K);
  const int tile_begin = (int)((int64_t)tiles_k * rank / S), tile_end = (int)((int64_t)tiles_k * (rank + 1) / S);
  const int T = tile_end - tile_begin;                        // tiles of this CTA's slice
  const int nrounds = (T + KL - 1) / KL;
  long long budget = 2000000000ll;

  // 1. the weight stream: round r of the slice -> ring slot r % kRing
  auto issue = [&](int r) {
    const int s = r % kRing;
    const int nt = min(KL, T - r * KL);
    const int64_t tile = mb * tiles_k + tile_begin + r * KL;
    const uint32_t dst = ob_ptx::smem_u32(wring + s * L::kRoundWeights);
    ob_ptx::mbar_expect_tx(bar_full(s), nt * kTileBytes);
    ob_ptx::bulk_load(dst, a.meta_tile + tile * OB_TILE_META_BYTES, nt * OB_TILE_META_BYTES, bar_full(s));
    ob_ptx::bulk_load(dst + KL * OB_TILE_META_BYTES, a.bits_tile + tile * OB_TILE_BITS_BYTES, nt * OB_TILE_BITS_BYTES, bar_full(s));
  };
  if (a.fresh_weights) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tid == 0) {
    for (int s = 0; s < kRing; ++s) { ob_ptx::mbar_init(bar_full(s), 1); ob_ptx::mbar_init(bar_empty(s), kThreads / 32); }
    ob_ptx::mbar_init(bar_recv, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (S > 1) ob_ptx::mbar_expect_tx(bar_recv, (uint32_t)L::kRecv);          // S slices x 128 / S rows x NP sums
    const int npre = min(nrounds, kRing);
    for (int r = 0; r < npre; ++r) issue(r);
  }
  __syncwarp();
  // Every CTA of the cluster announces that it runs; the matching wait stands right before the first store into
  // another CTA's shared memory, which must not be touched before that CTA has started.
  if (S > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may begin its own prologue
  asm volatile("griddepcontrol.wait;" ::: "memory");                // the previous kernel's results (the tokens) are complete
  OB_TRACE_EV(1);

  float acc[RG][NT][4];
#pragma unroll
  for (int rg = 0; rg < RG; ++rg)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[rg][nt][i] = 0.f;

  const int nvalid = (int)min((int64_t)NP, a.n - n0);
  // one token (n == 1) in the reference layout is the same contiguous vector as a token-major row; the
  // 16-byte loads of that form need an aligned base (token-major callers are checked on the host), any
  // other single token takes the element-wise path below
  const bool rows_contiguous = TM || (a.n == 1 && (reinterpret_cast<uintptr_t>(a.b) & 15) == 0);
  const bool quad_rows = !rows_contiguous && (a.n % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.b) & 7) == 0);
  const bool vec_rows = !rows_contiguous && (a.n % 8 == 0) && (nvalid == NP) && ((reinterpret_cast<uintptr_t>(a.b) & 15) == 0);

  // 2. tokens of one round: at most two 16-byte pieces per thread, fetched into registers, then scattered
  //    into tok[slot][tile][j][kk] = B[k0 + 128 tile + kk][n0 + j]. Rows j >= nvalid are never written.
  auto fetch_tokens = [&](int r, uint4 (&tv)[kPieces]) {
    const int ntile = min(KL, T - r * KL);
    const int64_t k0 = (int64_t)(tile_begin + r * KL) * OB_TILE_K;
#pragma unroll
    for (int i = 0; i < kPieces; ++i) {
      tv[i] = make_uint4(0, 0, 0, 0);
      const int idx = tid + kThreads * i;
      if (rows_contiguous) {
        // token j is contiguous along k: 16 pieces of 8 values per tile
        const int j = idx / (KL * 16), pc = idx % (KL * 16);
        if (j < nvalid && (pc >> 4) < ntile) tv[i] = __ldg(reinterpret_cast<const uint4*>(a.b + (n0 + j) * a.k + k0 + pc * 8));
      } else {
        const int kk = idx / NT, pc = idx % NT;               // k-row of the round, 8-token piece of that row
        if ((kk >> 7) < ntile) {
          if (vec_rows) {
            tv[i] = __ldg(reinterpret_cast<const uint4*>(a.b + (k0 + kk) * a.n + n0 + pc * 8));
          } else if (quad_rows) {
            uint2* h4 = reinterpret_cast<uint2*>(&tv[i]);     // n % 4 == 0: whole groups of four tokens
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4)
              if (8 * pc + 4 * q4 < nvalid) h4[q4] = __ldg(reinterpret_cast<const uint2*>(a.b + (k0 + kk) * a.n + n0 + 8 * pc + 4 * q4));
          } else {
            __half* h = reinterpret_cast<__half*>(&tv[i]);
#pragma unroll
            for (int jj = 0; jj < 8; ++jj)
              if (8 * pc + jj < nvalid) h[jj] = a.b[(k0 + kk) * a.n + n0 + 8 * pc + jj];
          }
        }
      }
    }
  };
  auto store_tokens = [&](int r, const uint4 (&tv)[kPieces]) {
    const int ntile = min(KL, T - r * KL);
    __half* sb = stok + (r % kRing) * (KL * NP * kTokStride);
#pragma unroll
    for (int i = 0; i < kPieces; ++i) {
      const int idx = tid + kThreads * i;
      if (rows_contiguous) {
        const int j = idx / (KL * 16), pc = idx % (KL * 16);
        if (j < nvalid && (pc >> 4) < ntile) *reinterpret_cast<uint4*>(&sb[((pc >> 4) * NP + j) * kTokStride + (pc & 15) * 8]) = tv[i];
      } else {
        const int kk = idx / NT, pc = idx % NT;
        const __half* h = reinterpret_cast<const __half*>(&tv[i]);
        if ((kk >> 7) < ntile) {
#pragma unroll
          for (int jj = 0; jj < 8; ++jj)
            if (8 * pc + jj < nvalid) sb[((kk >> 7) * NP + pc * 8 + jj) * kTokStride + (kk & 127)] = h[jj];
        }
      }
    }
  };

  // a span = the rounds that fit the ring; most decode shapes are a single span
  for (int r0 = 0; r0 < nrounds; r0 += kRing) {
    if (r0 > 0) __syncthreads();                              // the previous span's token buffers are free
    {
      uint4 tv[kRing][kPieces];
#pragma unroll
      for (int ri = 0; ri < kRing; ++ri)
        if (r0 + ri < nrounds) fetch_tokens(r0 + ri, tv[ri]);
#pragma unroll
      for (int ri = 0; ri < kRing; ++ri)
        if (r0 + ri < nrounds) store_tokens(r0 + ri, tv[ri]);
    }
    if (r0 == 0) OB_TRACE_EV(2);
    __syncthreads();                                          // tokens staged (and, first time, the mbarriers exist)
    if (r0 == 0) OB_TRACE_EV(3);

#pragma unroll 1
    for (int r = r0; r < min(nrounds, r0 + kRing); ++r) {
      const int s = r - r0;
      // every warp waits for every round: afterwards no copy of the slot is in flight
      ob_ptx::mbar_wait(bar_full(s), (r / kRing) & 1, budget, &g_decode_status, 101);
      if (r < 4) OB_TRACE_EV(8 + 2 * r);

      // 3. this warp's tile of the round: per 32-k block one token fragment feeds RG mma.sp
      if (r * KL + kl < T) {
        const uint8_t* wmeta = wring + s * L::kRoundWeights + kl * OB_TILE_META_BYTES;
        const uint8_t* wbits = wring + s * L::kRoundWeights + KL * OB_TILE_META_BYTES + kl * OB_TILE_BITS_BYTES;
        const __half* sb = stok + (s * KL + kl) * (NP * kTokStride);
        // this thread's token rows; columns beyond n read the zero row (their buffer rows are never written)
        const __half* trow[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) trow[nt] = (nt * 8 + g < nvalid) ? sb + (nt * 8 + g) * kTokStride : zrow;
#pragma unroll
        for (int p = 0; p < 2; ++p) {                         // pairs of 32-k blocks: one sign word per row
          uint32_t bf[2][NT][4];
#pragma unroll
          for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              // fragment register i: token column nt*8+g, k rows 2t+8i and 2t+8i+1 of the 32-k block
              const uint32_t* brow = reinterpret_cast<const uint32_t*>(trow[nt] + (2 * p + q) * 32);
#pragma unroll
              for (int i = 0; i < 4; ++i) bf[q][nt][i] = brow[t + 4 * i];
            }
          // RGC row groups at a time; consecutive MMAs go to different accumulators, so the next one
          // does not wait for the previous one
          constexpr int RGC = RG;
#pragma unroll
          for (int r0g = 0; r0g < RG; r0g += RGC) {
            uint2 mw[RGC];
            uint32_t wl[RGC], wh[RGC];
#pragma unroll
            for (int c = 0; c < RGC; ++c) {
              const int grp = rs * RG + r0g + c;              // 16-row group of the tile
              const int u = g + 8 * (t & 1) + 16 * grp;       // metadata lane of this thread
              mw[c] = *reinterpret_cast<const uint2*>(wmeta + u * 16 + p * 8);
              wl[c] = *reinterpret_cast<const uint32_t*>(wbits + (16 * grp + g) * 8 + p * 4);
              wh[c] = *reinterpret_cast<const uint32_t*>(wbits + (16 * grp + g + 8) * 8 + p * 4);
            }
#pragma unroll
            for (int q = 0; q < 2; ++q)
#pragma unroll
              for (int c = 0; c < RGC; ++c) {
                const int j1 = 8 * q + t, j2 = j1 + 4;
                const uint32_t af[4] = {expand_pair(wl[c], j1), expand_pair(wh[c], j1), expand_pair(wl[c], j2), expand_pair(wh[c], j2)};
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_sp_16832(acc[r0g + c][nt], af, bf[q][nt], q ? mw[c].y : mw[c].x);
              }
          }
        }
      }
      if (r < 4) OB_TRACE_EV(9 + 2 * r);
      // a slice longer than the ring: hand the weight slot back and refill it for the next span
      if (r + kRing < nrounds) {
        __syncwarp();
        if (lane == 0) ob_ptx::mbar_arrive(bar_empty(s));
        if (tid == 0) {
          ob_ptx::mbar_wait(bar_empty(s), (r / kRing) & 1, budget, &g_decode_status, 102);
          issue(r + kRing);
        }
        __syncwarp();
      }
    }
  }

  OB_TRACE_EV(4);
  // 4. the KL partial sums of the CTA meet in shared memory: the ring is drained (every warp has seen
  //    every round land), so it serves as the buffer red[tile lane][row][token]
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem);
#pragma unroll
  for (int rg = 0; rg < RG; ++rg)
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      const int row = (rs * RG + rg) * 16 + g + 8 * hrow;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        *reinterpret_cast<float2*>(&red[(kl * 128 + row) * NP + nt * 8 + 2 * t]) = make_float2(acc[rg][nt][2 * hrow], acc[rg][nt][2 * hrow + 1]);
    }
  __syncthreads();

  auto finish = [&](int64_t row, int j, float sum, float scale, float bias) {
    sum = __fmul_rn(sum, scale);                              // two roundings, like the other kernels' epilogues
    if (a.bias) sum = __fadd_rn(sum, bias);
    if (j < nvalid) {
      const int64_t o = TM ? (n0 + j) * a.m + row : row * a.n + n0 + j;
      if constexpr (sizeof(OutT) == 2) static_cast<__half*>(a.d)[o] = __float2half_rn(sum);
      else static_cast<float*>(a.d)[o] = sum;
    }
  };
  // each thread adds the lanes for NT groups of four consecutive tokens of one row
  constexpr int kQuads = 128 * NP / 4;                        // = NT * kThreads
  const int rows_per = 128 / S;                               // S is a power of two
  if (S > 1) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");   // all CTAs of the cluster have started
#pragma unroll
  for (int i = 0; i < kQuads / kThreads; ++i) {
    const int x = tid + i * kThreads;
    float4 v = *reinterpret_cast<const float4*>(&red[4 * x]);
#pragma unroll
    for (int l = 1; l < KL; ++l) {
      const float4 w = *reinterpret_cast<const float4*>(&red[l * 128 * NP + 4 * x]);
      v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
    }
    const int row = 4 * x / NP, j = 4 * x % NP;
    if (S == 1) {
      // no other CTA shares these rows
      const int64_t grow = mb * 128 + row;
      const float scale = a.scale ? __half2float(a.scale[grow]) : 1.f, bias = a.bias ? __half2float(a.bias[grow]) : 0.f;
      finish(grow, j, v.x, scale, bias); finish(grow, j + 1, v.y, scale, bias);
      finish(grow, j + 2, v.z, scale, bias); finish(grow, j + 3, v.w, scale, bias);
    } else {
      // 5. one 16-byte push to the CTA that owns the row: CTA q of the cluster owns rows [q * 128/S, (q+1) * 128/S)
      //    The store completes on the owner's mbarrier: data and signal travel together, no cluster-wide barrier
      //    stands between the last MMA and the sum.
      const uint32_t owner = (uint32_t)(row / rows_per);
      const uint32_t local = ob_ptx::smem_u32(s_recv) + (uint32_t)(((rank * rows_per + row % rows_per) * NP + j) * 4);
      asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                   ::"r"(ob_ptx::map_to_cta(local, owner)), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(ob_ptx::map_to_cta(bar_recv, owner)) : "memory");
    }
  }
  if (S == 1) { OB_TRACE_EV(7); return; }
  OB_TRACE_EV(5);
  // the per-row constants of this thread's outputs, fetched while the sums travel
  constexpr int kOut = (128 * NP / 2 + kThreads - 1) / kThreads;   // outputs per thread at S = 2, the most
  float sc[kOut], bs[kOut];
#pragma unroll
  for (int i = 0; i < kOut; ++i) {
    const int e = tid + i * kThreads;
    sc[i] = 1.f; bs[i] = 0.f;
    if (e < rows_per * NP) {
      const int rr = TM ? e % rows_per : e / NP;
      const int64_t row = mb * 128 + rank * rows_per + rr;
      if (a.scale) sc[i] = __half2float(a.scale[row]);
      if (a.bias) bs[i] = __half2float(a.bias[row]);
    }
  }
  ob_ptx::mbar_wait(bar_recv, 0, budget, &g_decode_status, 103);   // all S slices of this CTA's rows are here
  OB_TRACE_EV(6);

  // 6. fixed-order sum of the S slices from this CTA's own shared memory
#pragma unroll
  for (int i = 0; i < kOut; ++i) {
    const int e = tid + i * kThreads;
    if (e < rows_per * NP) {
      // consecutive threads walk the fastest output dimension: tokens of a row (m x n), rows of a token (n x m)
      const int rr = TM ? e % rows_per : e / NP, j = TM ? e / rows_per : e % NP;
      float sum = 0.f;
      for (int sl = 0; sl < S; ++sl) sum += s_recv[(sl * rows_per + rr) * NP + j];
      finish(mb * 128 + rank * rows_per + rr, j, sum, sc[i], bs[i]);
    }
  }
  OB_TRACE_EV(7);
}

template <int NT, typename OutT, bool TM>
cudaError_t launch(const DecodeArgs& a, int S, cudaStream_t stream) {
  using L = DecodeCfg<NT>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(ob_gemm_decode_kernel<NT, OutT, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(a.m / 128), (unsigned)S, (unsigned)((a.n + NT * 8 - 1) / (NT * 8)));
  cfg.blockDim = dim3(L::kThreads);
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
  return cudaLaunchKernelEx(&cfg, ob_gemm_decode_kernel<NT, OutT, TM>, a);
}

}  // namespace

namespace ob {

namespace {
// K split over a cluster of S CTAs. A CTA multiplies its slice in rounds of `lanes` tiles, and an SM
// holds two CTAs: S minimises rounds x CTAs per SM among the splits that keep the grid one wave.
int pick_split(int64_t m, int64_t k, int lanes) {
  const int64_t tiles_k = k / OB_TILE_K, row_blocks = m / 128;
  const int sms = ob::sm_count();
  int best = 1;
  long long best_cost = LLONG_MAX;
  for (int S = 1; S <= 8; S *= 2) {
    if (S > 1 && (row_blocks * S > 2 * sms || tiles_k < S)) break;
    const long long T = (tiles_k + S - 1) / S, rounds = (T + lanes - 1) / lanes, per_sm = (row_blocks * S + sms - 1) / sms;
    if (rounds * per_sm <= best_cost) { best = S; best_cost = rounds * per_sm; }   // ties: more CTAs stream
  }
  // tuning knob for experiments
  static const int forced = [] { const char* v = getenv("ONEBIT_DECODE_SPLIT"); return v ? atoi(v) : 0; }();
  if ((forced == 1 || forced == 2 || forced == 4 || forced == 8) && forced <= tiles_k) best = forced;
  return best;
}
template <bool TM>
cudaError_t dispatch(const DecodeArgs& a, int out_type, cudaStream_t stream) {
  const bool two = (a.n > 8);
  const int S = pick_split(a.m, a.k, two ? DecodeCfg<2>::KL : DecodeCfg<1>::KL);
  if (out_type == OB_OUT_F16) return two ? launch<2, __half, TM>(a, S, stream) : launch<1, __half, TM>(a, S, stream);
  return two ? launch<2, float, TM>(a, S, stream) : launch<1, float, TM>(a, S, stream);
}
}  // namespace

cudaError_t launch_gemm_decode(const void* bits_tile, const void* meta_tile, const void* scale, const void* b,
                               void* d, int64_t m, int64_t n, int64_t k, int out_type, bool fresh_weights,
                               cudaStream_t stream) {
  DecodeArgs a{static_cast<const uint8_t*>(bits_tile), static_cast<const uint8_t*>(meta_tile),
               static_cast<const __half*>(scale), nullptr, static_cast<const __half*>(b), d, m, n, k, fresh_weights ? 1 : 0};
  return dispatch<false>(a, out_type, stream);
}

cudaError_t launch_gemm_decode_tokens(const void* bits_tile, const void* meta_tile, const void* scale, const void* bias,
                                      const void* x, void* y, int64_t m, int64_t n, int64_t k, int out_type,
                                      bool fresh_weights, cudaStream_t stream) {
  DecodeArgs a{static_cast<const uint8_t*>(bits_tile), static_cast<const uint8_t*>(meta_tile),
               static_cast<const __half*>(scale), static_cast<const __half*>(bias), static_cast<const __half*>(x), y, m, n, k,
               fresh_weights ? 1 : 0};
  return dispatch<true>(a, out_type, stream);
}

// Reads and clears the decode kernel's wait status on the current device (0 = no wait gave up).
cudaError_t read_decode_status(int* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_decode_status, sizeof(int));
  if (e != cudaSuccess || *out == 0) return e;
  const int zero = 0;
  return cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
}

}  // namespace ob

#ifdef OB_TRACE
extern "C" int onebit_debug_read_trace_decode(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_trace_dec, sizeof(long long) * 4 * 16);
}
#endif
