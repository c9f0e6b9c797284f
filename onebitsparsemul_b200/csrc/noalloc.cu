// onebit_sparse_matmul_static: the stateless GEMM for callers that must not allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits -- an inference server whose own pool
// already holds all of the GPU's memory (a fresh cudaMalloc there fails or fragments the pool), a
// latency-critical decode loop that cannot afford cudaMalloc's implicit device-wide synchronisation,
// or a host that forbids allocation after start-up. The other stateless entry point either takes a
// caller-provided workspace or grows a cached cudaMalloc'ed one; this one does neither. Its relayout
// target (the tile-ordered copy of the weights that the GEMM kernel reads) is a fixed array that is
// part of the library image: a GPU holds these ~8 MiB from the moment the driver loads this part of
// the library on it until the process exits. With CUDA's default lazy module loading that moment is the
// first call of this function on the device (the address look-up below), with eager loading it is the
// creation of the context; so the first call per device belongs into start-up, as a warm-up, while device
// memory is still to be had -- it can fail like an allocation. Every later call touches no allocator.
//
// Limits and rules
//   * m * k <= ONEBIT_STATIC_MAX_WEIGHTS (4096 x 11008, the largest 7B-class decode layer); larger
//     problems are rejected with ONEBIT_ERR_WORKSPACE and a message -- nothing is launched.
//   * Shapes must be tile-shaped (m % 128 == 0, k % 128 == 0); the GEMM always runs on the split-K
//     cluster kernel (any n; meant for few tokens).
//   * The first call on each device looks up the array's device address (once per device, with that
//     device current) and thereby may make the driver load the module and reserve the array. Make that
//     first call at start-up, outside any stream capture.
//   * All calls on a device share the one array, and it keeps the previous call's contents. Every
//     byte the GEMM reads is rewritten by the relayout of the same call, so nothing needs clearing,
//     but two calls whose kernels overlap on the GPU (different streams, no dependency) race on it:
//     serialise them.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on the first call or later (the
//     test watches cudaMemGetInfo across the later calls).
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/onebit_sparse_tensor.h"
#include "formats.h"
#include "kernels.h"

namespace {

constexpr size_t kBitsBytes = ONEBIT_STATIC_MAX_WEIGHTS / 16;   // 2 818 048, a multiple of 256
constexpr size_t kMetaBytes = ONEBIT_STATIC_MAX_WEIGHTS / 8;    // 5 636 096, a multiple of 256
static_assert(kBitsBytes % 256 == 0 && kMetaBytes % 256 == 0, "static scratch halves must stay 256-byte aligned");

// In host code this name is only a handle for the runtime's symbol table, never a device address:
// the address each device gave the array is fetched with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kBitsBytes + kMetaBytes];

std::mutex g_mu;
unsigned char* g_scratch_addr[64] = {};

thread_local char g_msg[256] = "";

}  // namespace

// Defined in api.cu: stores the message that onebit_last_error() returns for this thread.
namespace ob { void set_last_error(const char* msg); }

extern "C" int onebit_sparse_matmul_static(const void* a_bits, const void* b, void* d, const void* e_meta, const void* scale,
                                           int64_t m, int64_t n, int64_t k, int out_type, int meta_dialect, void* stream) {
  auto fail = [](int code, const char* msg) { ob::set_last_error(msg); return code; };
  if (!a_bits || !b || !d || !e_meta) return fail(ONEBIT_ERR_NULL, "null operand pointer");
  if (m <= 0 || n <= 0 || k <= 0 || m % OB_TILE_M != 0 || k % OB_TILE_K != 0)
    return fail(ONEBIT_ERR_SHAPE, "onebit_sparse_matmul_static needs m % 128 == 0, k % 128 == 0, n >= 1");
  if (meta_dialect != OB_META_PYTHON && meta_dialect != OB_META_CUTLASS) return fail(ONEBIT_ERR_ARG, "unknown metadata order");
  if (out_type != OB_OUT_F32 && out_type != OB_OUT_F16) return fail(ONEBIT_ERR_ARG, "unknown output type");
  // m and k are bounded one by one first, so that the product cannot wrap
  if (m > ONEBIT_STATIC_MAX_WEIGHTS / OB_TILE_K || k > ONEBIT_STATIC_MAX_WEIGHTS / OB_TILE_M ||
      (uint64_t)m * (uint64_t)k > (uint64_t)ONEBIT_STATIC_MAX_WEIGHTS) {
    snprintf(g_msg, sizeof(g_msg),
             "onebit_sparse_matmul_static: m*k = %lld exceeds the built-in scratch (%lld weights); use "
             "onebit_sparse_matmul_ex with a workspace", (long long)((double)m * (double)k), (long long)ONEBIT_STATIC_MAX_WEIGHTS);
    return fail(ONEBIT_ERR_WORKSPACE, g_msg);
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ONEBIT_ERR_CUDA, cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(ONEBIT_ERR_ARG, "device ordinal not supported");
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_scratch_addr[dev]) {
      // once per device, with that device current: the array's address on THIS device
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || !p) {
        snprintf(g_msg, sizeof(g_msg), "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        return fail(ONEBIT_ERR_CUDA, g_msg);
      }
      g_scratch_addr[dev] = static_cast<unsigned char*>(p);
    }
    scratch = g_scratch_addr[dev];
  }
  void* bits_tile = scratch;
  void* meta_tile = scratch + kBitsBytes;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  e = ob::launch_relayout(a_bits, e_meta, meta_dialect, m, k, bits_tile, meta_tile, st);
  if (e != cudaSuccess) return fail(ONEBIT_ERR_CUDA, cudaGetErrorString(e));
  e = ob::launch_gemm_decode(bits_tile, meta_tile, scale, b, d, m, n, k, out_type, /*fresh_weights=*/true, st);
  if (e != cudaSuccess) return fail(ONEBIT_ERR_CUDA, cudaGetErrorString(e));
  return ONEBIT_OK;
}
