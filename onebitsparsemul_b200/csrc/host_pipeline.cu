// onebit_matmul_packed_host: the GEMM for callers whose tokens and results live in HOST memory.
//
// The reference's Python entry point does exactly this by accident -- it allocates C on the CPU and
// hands its pointer to the kernel (onebit_sparse_mul/__init__.py:12-15). Here the transfers are part
// of the call and are overlapped with the compute: the token matrix is cut into column panels;
// panel p+1 travels host -> device (pitched copy) while panel p is multiplied and panel p-1 travels
// device -> host. PCIe is full duplex, so a call costs about max(H2D, D2H) instead of
// H2D + GEMM + D2H. Three device staging slots rotate; three internal streams per device carry the
// three legs; the caller's stream is joined at both ends with events, so the call is asynchronous for
// the host like every other entry point.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "../../include/onebit_sparse_tensor.h"
#include "formats.h"
#include "kernels.h"

namespace ob { void set_last_error(const char* msg); }

namespace {

constexpr int kSlots = 3;
constexpr int kMaxPanels = 64;

struct DevicePipes {
  bool ready = false;
  cudaStream_t in = nullptr, compute = nullptr, out = nullptr;
  cudaEvent_t start = nullptr, done = nullptr;
  cudaEvent_t loaded[kSlots] = {}, computed[kSlots] = {}, drained[kSlots] = {};
};
std::mutex g_mu;
DevicePipes g_pipes[64];

int fail(int code, const char* msg) { ob::set_last_error(msg); return code; }
int cuda_fail(cudaError_t e, const char* what) {
  static thread_local char buf[256];
  snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
  return fail(ONEBIT_ERR_CUDA, buf);
}

size_t round256(size_t x) { return (x + 255) & ~size_t(255); }

int64_t panel_width(int64_t n) {
  // Whole 256-token tiles. Measured on PCIe Gen5: pitched copies want rows of >= 2 KiB (1024 tokens) and
  // a handful of panels; more, narrower panels lose more to the DMA engines than the shorter pipeline
  // fill and drain win back. ONEBIT_HOST_PANELS overrides the panel count for experiments.
  static const int forced = [] { const char* v = getenv("ONEBIT_HOST_PANELS"); return v ? atoi(v) : 0; }();
  auto up256 = [](int64_t x) { return (x + 255) / 256 * 256; };
  if (forced > 0) return std::max<int64_t>(256, up256((n + forced - 1) / forced));
  int64_t w = std::max<int64_t>(2048, up256((n + 7) / 8));      // at most 8 panels, at least 2048 tokens wide
  if (n >= 512) w = std::min(w, up256((n + 1) / 2));             // but at least two panels to overlap anything
  return std::max<int64_t>(256, w);
}

}  // namespace

extern "C" size_t onebit_host_workspace_bytes(int64_t m, int64_t n, int64_t k, int out_type) {
  const int64_t np = std::min(panel_width(n), (n + 7) / 8 * 8);
  const size_t esz = out_type == ONEBIT_OUT_F16 ? 2 : 4;
  return kSlots * (round256((size_t)k * np * 2) + round256((size_t)m * np * esz));
}

extern "C" int onebit_matmul_packed_host(const void* bits_tile, const void* meta_tile, const void* scale,
                                         const void* b_host, void* d_host, int64_t m, int64_t n, int64_t k, int out_type,
                                         void* workspace, size_t workspace_bytes, void* stream) {
  if (!bits_tile || !meta_tile || !b_host || !d_host || !workspace) return fail(ONEBIT_ERR_NULL, "null operand or workspace pointer");
  if (m <= 0 || k <= 0 || n < 8 || m % OB_TILE_M || k % OB_TILE_K || n % 8)
    return fail(ONEBIT_ERR_SHAPE, "onebit_matmul_packed_host needs m % 128 == 0, k % 128 == 0, n % 8 == 0, n >= 8");
  if (out_type != ONEBIT_OUT_F32 && out_type != ONEBIT_OUT_F16) return fail(ONEBIT_ERR_ARG, "unknown output type");
  if (workspace_bytes < onebit_host_workspace_bytes(m, n, k, out_type) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(ONEBIT_ERR_WORKSPACE, "workspace too small (see onebit_host_workspace_bytes) or not 256-byte aligned");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(ONEBIT_ERR_ARG, "device ordinal not supported");
  // The lock is held for the whole enqueue: the per-device streams and events are shared, and records and
  // waits of two interleaved calls would pair up wrongly.
  std::lock_guard<std::mutex> lk(g_mu);
  DevicePipes* P = &g_pipes[dev];
  {
    if (!P->ready) {
      cudaStream_t* ss[3] = {&P->in, &P->compute, &P->out};
      for (auto s : ss) if ((e = cudaStreamCreateWithFlags(s, cudaStreamNonBlocking)) != cudaSuccess) return cuda_fail(e, "cudaStreamCreate");
      cudaEvent_t* one[2] = {&P->start, &P->done};
      for (auto ev : one) if ((e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
      for (int i = 0; i < kSlots; ++i) {
        cudaEvent_t* three[3] = {&P->loaded[i], &P->computed[i], &P->drained[i]};
        for (auto ev : three) if ((e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
      }
      P->ready = true;
    }
  }
  const size_t esz = out_type == ONEBIT_OUT_F16 ? 2 : 4;
  const int64_t np = std::min(panel_width(n), (n + 7) / 8 * 8);
  const int64_t panels = (n + np - 1) / np;
  if (panels > kMaxPanels) return fail(ONEBIT_ERR_SHAPE, "too many token panels");
  const size_t b_slot = round256((size_t)k * np * 2), c_slot = round256((size_t)m * np * esz);
  char* ws = static_cast<char*>(workspace);
  auto b_dev = [&](int s) { return ws + (size_t)s * (b_slot + c_slot); };
  auto c_dev = [&](int s) { return ws + (size_t)s * (b_slot + c_slot) + b_slot; };

  cudaStream_t user = static_cast<cudaStream_t>(stream);
  // the internal streams start after everything already queued on the caller's stream
  if ((e = cudaEventRecord(P->start, user)) != cudaSuccess) return cuda_fail(e, "cudaEventRecord");
  cudaStreamWaitEvent(P->in, P->start, 0);
  cudaStreamWaitEvent(P->compute, P->start, 0);
  cudaStreamWaitEvent(P->out, P->start, 0);
  // the caller's stream continues when all three internal streams have run dry: the last result panel is
  // home and nothing reads the slots any more. Also used on the error paths, so that whatever was queued
  // before a failure is still ordered before the caller's later work.
  auto join = [&] {
    cudaStream_t legs[3] = {P->in, P->compute, P->out};
    for (cudaStream_t leg : legs) {
      cudaEventRecord(P->done, leg);
      cudaStreamWaitEvent(user, P->done, 0);
    }
  };

  for (int64_t p = 0; p < panels; ++p) {
    const int s = (int)(p % kSlots);
    const int64_t c0 = p * np, w = std::min(np, n - c0);
    // host -> device, pitched: k rows of w tokens. The slot's previous user -- panel p - kSlots, or a panel of
    // the previous call on this device, which may have come from another stream with the same workspace --
    // must have been multiplied (an event that was never recorded does not hold anything up)
    cudaStreamWaitEvent(P->in, P->computed[s], 0);
    e = cudaMemcpy2DAsync(b_dev(s), (size_t)w * 2, static_cast<const char*>(b_host) + (size_t)c0 * 2, (size_t)n * 2,
                          (size_t)w * 2, (size_t)k, cudaMemcpyHostToDevice, P->in);
    if (e != cudaSuccess) { join(); return cuda_fail(e, "cudaMemcpy2DAsync(H2D)"); }
    cudaEventRecord(P->loaded[s], P->in);
    // GEMM on the panel (the dispatcher picks the kernel for its width)
    cudaStreamWaitEvent(P->compute, P->loaded[s], 0);
    cudaStreamWaitEvent(P->compute, P->drained[s], 0);      // and its result must have left the slot
    const int rc = onebit_matmul_packed(bits_tile, meta_tile, scale, b_dev(s), c_dev(s), m, w, k, out_type, ONEBIT_KERNEL_AUTO, P->compute);
    if (rc != ONEBIT_OK) { join(); return rc; }
    cudaEventRecord(P->computed[s], P->compute);
    // device -> host, pitched
    cudaStreamWaitEvent(P->out, P->computed[s], 0);
    e = cudaMemcpy2DAsync(static_cast<char*>(d_host) + (size_t)c0 * esz, (size_t)n * esz, c_dev(s), (size_t)w * esz,
                          (size_t)w * esz, (size_t)m, cudaMemcpyDeviceToHost, P->out);
    if (e != cudaSuccess) { join(); return cuda_fail(e, "cudaMemcpy2DAsync(D2H)"); }
    cudaEventRecord(P->drained[s], P->out);
  }
  join();
  return ONEBIT_OK;
}

// Pitched copy between host and device, direction from the pointers; see the header.
extern "C" int onebit_copy_2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                                    size_t rows, void* stream) {
  if (!dst || !src) return fail(ONEBIT_ERR_NULL, "null pointer");
  if (row_bytes == 0 || rows == 0) return ONEBIT_OK;
  if (dst_pitch < row_bytes || src_pitch < row_bytes) return fail(ONEBIT_ERR_ARG, "a pitch is smaller than a row");
  cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, rows, cudaMemcpyDefault, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy2DAsync");
  return ONEBIT_OK;
}
