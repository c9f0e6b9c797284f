// The C ABI of libonebitmul (declared in include/onebit_sparse_tensor.h) and the host dispatcher.
//
// Counterpart of the reference's csrc/kernel_lib.cu:23-97: where that file wraps the pointers into
// CUTLASS TensorRefs and launches one templated SparseGemm, this one validates the shape, brings
// reference-ordered operands into tile order (relayout.cu) and picks one of two hand-written
// kernels by shape: the split-K cluster kernel for few tokens (gemm_decode.cu) or the TMA +
// tcgen05.mma.sp kernel (gemm_prefill_sm100.cu). There is no CPU path: without a CUDA device every
// entry point fails with ONEBIT_ERR_CUDA.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "../../include/onebit_sparse_tensor.h"
#include "formats.h"
#include "kernels.h"

static_assert((int)ONEBIT_META_PYTHON == (int)OB_META_PYTHON && (int)ONEBIT_META_CUTLASS == (int)OB_META_CUTLASS, "enum drift");
static_assert((int)ONEBIT_OUT_F32 == (int)OB_OUT_F32 && (int)ONEBIT_OUT_F16 == (int)OB_OUT_F16, "enum drift");
static_assert((int)ONEBIT_DENSE_F16 == (int)OB_DENSE_F16 && (int)ONEBIT_DENSE_BF16 == (int)OB_DENSE_BF16 && (int)ONEBIT_DENSE_I32 == (int)OB_DENSE_I32,
              "enum drift");

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(ONEBIT_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

size_t round256(size_t x) { return (x + 255) & ~size_t(255); }

bool tiled_shape(int64_t m, int64_t k) { return m > 0 && k > 0 && m % OB_TILE_M == 0 && k % OB_TILE_K == 0; }

// Per-device state owned by the library: the status word of the tensor-memory kernels and the relayout
// scratch of the stateless entry points when the caller passes no workspace. The scratch is grown on
// demand and never freed or shrunk while the process lives: a block that was outgrown may still be read by
// launches already queued, so it is only retired. Calls that share it are ordered on the GPU by `last_use`
// (recorded after each call's GEMM, waited on before the next call's relayout), whatever streams they use.
struct DeviceScratch {
  void* buf = nullptr;
  size_t bytes = 0;
  int* status = nullptr;
  cudaEvent_t last_use = nullptr;
  int sms = 0;
};
std::mutex g_mu;           // guards the fields of g_scratch
std::mutex g_scratch_mu;   // held for the whole enqueue of a call that uses the library-owned scratch block
DeviceScratch g_scratch[64];

int current_device(int* dev) {
  cudaError_t e = cudaGetDevice(dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (*dev < 0 || *dev >= 64) return fail(ONEBIT_ERR_ARG, "device ordinal %d not supported", *dev);
  return ONEBIT_OK;
}

int get_status_word(int** out) {
  int dev = 0;
  if (int rc = current_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceScratch& s = g_scratch[dev];
  if (!s.status) {
    cudaError_t e = cudaMalloc(&s.status, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(status)");
    e = cudaMemset(s.status, 0, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(status)");
  }
  *out = s.status;
  return ONEBIT_OK;
}

// Called with g_scratch_mu held. Makes the device's scratch at least `bytes` large.
int grow_scratch_locked(DeviceScratch& s, size_t bytes) {
  if (!s.last_use) {
    cudaError_t e = cudaEventCreateWithFlags(&s.last_use, cudaEventDisableTiming);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
  }
  if (s.bytes >= bytes) return ONEBIT_OK;
  void* fresh = nullptr;
  cudaError_t e = cudaMalloc(&fresh, bytes);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(scratch)");
  s.buf = fresh;      // the outgrown block stays allocated: queued launches may still read it
  s.bytes = bytes;
  return ONEBIT_OK;
}

// Which few-token kernel serves ONEBIT_KERNEL_DECODE. Both stream the same tile-ordered operands with the same
// cluster split-K; the tensor-memory form (gemm_decode_sm100.cu) is faster except for the smallest calls, where
// its longer start-up (tensor-memory allocation, more hand-overs before the first MMA) outweighs its cheaper
// multiply phase: measured 4.9 against 4.3 us at 4096 x 4096 with up to 8 tokens, 7.6 against 8.5 us at
// 11008 x 4096, 9.3 against 15.5 us there with 16 tokens. ONEBIT_DECODE_VARIANT=1 / 2 in the environment forces the
// warp-level mma.sp form / the tensor-memory form.
bool use_legacy_decode(int64_t m, int64_t n, int64_t k) {
  static const int forced = [] { const char* v = getenv("ONEBIT_DECODE_VARIANT"); return v ? atoi(v) : 0; }();
  if (forced == 1) return true;
  if (forced == 2) return false;
  // measured (graph replay, us): 4096 x 4096, n = 1 / 8: 3.8 / 4.1 against 4.9 / 5.0; 4096 x 11008, n = 1: 6.9 against 7.3
  return (n <= 8 && m * k <= 4096ll * 4096ll) || (n == 1 && m <= 4096 && m * k <= 4096ll * 11008ll);
}

int check_dialect_rows(int dialect, int64_t m) {
  if (dialect != OB_META_PYTHON && dialect != OB_META_CUTLASS) return fail(ONEBIT_ERR_ARG, "unknown metadata order %d", dialect);
  if (m % ob_meta_row_granule(dialect) != 0)
    return fail(ONEBIT_ERR_SHAPE, "m = %lld must be a multiple of %d for this metadata order", (long long)m,
                ob_meta_row_granule(dialect));
  return ONEBIT_OK;
}

int matmul_packed_impl(const void* bits_tile, const void* meta_tile, const void* scale, const void* b, void* d,
                       int64_t m, int64_t n, int64_t k, int out_type, int kernel, cudaStream_t stream) {
  // unless the caller vouches for the age of the packed weights, the few-token kernel requests them only
  // after the kernel before it in the stream has completed
  const bool fresh_weights = (kernel & ONEBIT_KERNEL_STABLE_WEIGHTS) == 0;
  kernel &= ~ONEBIT_KERNEL_STABLE_WEIGHTS;
  if (!bits_tile || !meta_tile || !b || !d) return fail(ONEBIT_ERR_NULL, "null operand pointer");
  if (!tiled_shape(m, k) || n < 1)
    return fail(ONEBIT_ERR_SHAPE, "tile-ordered GEMM needs m %% 128 == 0, k %% 128 == 0, n >= 1 (got m=%lld n=%lld k=%lld)",
                (long long)m, (long long)n, (long long)k);
  if (out_type != OB_OUT_F32 && out_type != OB_OUT_F16) return fail(ONEBIT_ERR_ARG, "unknown output type %d", out_type);
  // Up to 16 tokens, and up to 32 on matrices of at most 8192 rows (two passes of the few-token kernel still beat
  // the tile kernels there: 7.6 against 12 us at 4096 x 4096, 19 against 23 us at 8192 x 8192; at 11008 rows the
  // tile kernel fills the chip and wins, 14.5 against 20 us): the few-token kernel. More tokens: the tile kernels.
  if (kernel == ONEBIT_KERNEL_AUTO)
    kernel = ((n > 32 || (n > 16 && m > 8192)) && ob::prefill_supported(m, n, k)) ? ONEBIT_KERNEL_PREFILL : ONEBIT_KERNEL_DECODE;
  cudaError_t e;
  if (kernel == ONEBIT_KERNEL_PREFILL) {
    if (!ob::prefill_supported(m, n, k))
      return fail(ONEBIT_ERR_SHAPE, "the tensor-memory kernel needs n %% 8 == 0 (got n=%lld)", (long long)n);
    int* status = nullptr;
    if (int rc = get_status_word(&status)) return rc;
    e = ob::launch_gemm_prefill(bits_tile, meta_tile, scale, b, d, m, n, k, out_type, status, stream);
    if (e != cudaSuccess) return cuda_fail(e, "tensor-memory GEMM launch");
  } else if (kernel == ONEBIT_KERNEL_DECODE) {
    e = use_legacy_decode(m, n, k) ? ob::launch_gemm_decode(bits_tile, meta_tile, scale, b, d, m, n, k, out_type, fresh_weights, stream)
                            : ob::launch_gemm_fewtok(bits_tile, meta_tile, scale, nullptr, b, d, m, n, k, out_type, false, fresh_weights, stream);
    if (e != cudaSuccess) return cuda_fail(e, "decode GEMM launch");
  } else {
    return fail(ONEBIT_ERR_ARG, "unknown kernel selector %d", kernel);
  }
  return ONEBIT_OK;
}

}  // namespace

namespace ob {
// lets the other translation units of the library report through onebit_last_error()
void set_last_error(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceScratch& s = g_scratch[dev];
  if (s.sms == 0 && cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) s.sms = 0;
  return s.sms > 0 ? s.sms : 148;
}
}  // namespace ob

extern "C" {

const char* onebit_last_error(void) { return g_err; }

size_t onebit_packed_bits_bytes(int64_t m, int64_t k) { return (size_t)(m * k / 16); }
size_t onebit_packed_meta_bytes(int64_t m, int64_t k) { return (size_t)(m * k / 8); }
size_t onebit_workspace_bytes(int64_t m, int64_t k) {
  return round256(onebit_packed_bits_bytes(m, k)) + round256(onebit_packed_meta_bytes(m, k));
}

int onebit_relayout(const void* a_bits, const void* e_meta, int meta_dialect, int64_t m, int64_t k, void* bits_tile,
                    void* meta_tile, void* stream) {
  if (!a_bits || !e_meta || !bits_tile || !meta_tile) return fail(ONEBIT_ERR_NULL, "null operand pointer");
  if (!tiled_shape(m, k)) return fail(ONEBIT_ERR_SHAPE, "tile order needs m %% 128 == 0 and k %% 128 == 0 (got m=%lld k=%lld)", (long long)m, (long long)k);
  if (int rc = check_dialect_rows(meta_dialect, m)) return rc;
  cudaError_t e = ob::launch_relayout(a_bits, e_meta, meta_dialect, m, k, bits_tile, meta_tile, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? ONEBIT_OK : cuda_fail(e, "relayout launch");
}

int onebit_matmul_packed(const void* bits_tile, const void* meta_tile, const void* scale, const void* b, void* d,
                         int64_t m, int64_t n, int64_t k, int out_type, int kernel, void* stream) {
  return matmul_packed_impl(bits_tile, meta_tile, scale, b, d, m, n, k, out_type, kernel, static_cast<cudaStream_t>(stream));
}

int onebit_linear_tokens(const void* bits_tile, const void* meta_tile, const void* scale, const void* bias, const void* x,
                         void* y, int64_t m, int64_t n, int64_t k, int out_type, int kernel, void* stream) {
  if (!bits_tile || !meta_tile || !x || !y) return fail(ONEBIT_ERR_NULL, "null operand pointer");
  if (!tiled_shape(m, k) || n < 1)
    return fail(ONEBIT_ERR_SHAPE, "token-major GEMM needs m %% 128 == 0, k %% 128 == 0, n >= 1 (got m=%lld n=%lld k=%lld)",
                (long long)m, (long long)n, (long long)k);
  if (out_type != OB_OUT_F32 && out_type != OB_OUT_F16) return fail(ONEBIT_ERR_ARG, "unknown output type %d", out_type);
  if (reinterpret_cast<uintptr_t>(x) & 15) return fail(ONEBIT_ERR_ARG, "x must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool fresh_weights = (kernel & ONEBIT_KERNEL_STABLE_WEIGHTS) == 0;
  kernel &= ~ONEBIT_KERNEL_STABLE_WEIGHTS;
  if (kernel == ONEBIT_KERNEL_AUTO)
    kernel = (n > 16 && ob::prefill_tokens_supported(m, n, k)) ? ONEBIT_KERNEL_PREFILL : ONEBIT_KERNEL_DECODE;
  cudaError_t e;
  if (kernel == ONEBIT_KERNEL_PREFILL) {
    if (!ob::prefill_tokens_supported(m, n, k))
      return fail(ONEBIT_ERR_SHAPE, "the token-major tensor-memory kernel needs m %% 256 == 0 (got m=%lld)", (long long)m);
    int* status = nullptr;
    if (int rc = get_status_word(&status)) return rc;
    e = ob::launch_gemm_prefill_tokens(bits_tile, meta_tile, scale, bias, x, y, m, n, k, out_type, status, st);
    if (e != cudaSuccess) return cuda_fail(e, "token-major tensor-memory GEMM launch");
  } else if (kernel == ONEBIT_KERNEL_DECODE) {
    e = use_legacy_decode(m, n, k) ? ob::launch_gemm_decode_tokens(bits_tile, meta_tile, scale, bias, x, y, m, n, k, out_type, fresh_weights, st)
                            : ob::launch_gemm_fewtok(bits_tile, meta_tile, scale, bias, x, y, m, n, k, out_type, true, fresh_weights, st);
    if (e != cudaSuccess) return cuda_fail(e, "token-major decode GEMM launch");
  } else {
    return fail(ONEBIT_ERR_ARG, "unknown kernel selector %d", kernel);
  }
  return ONEBIT_OK;
}

int onebit_matmul_packed_scatter(const void* bits_tile, const void* meta_tile, const void* scale, const void* b, void* d,
                                 void* const* extra_dst, int n_extra, int64_t m, int64_t n, int64_t k, void* stream) {
  if (!bits_tile || !meta_tile || !b || !d) return fail(ONEBIT_ERR_NULL, "null operand pointer");
  if (n_extra < 0 || n_extra > 7) return fail(ONEBIT_ERR_ARG, "n_extra = %d, at most 7 extra destinations", n_extra);
  if (n_extra > 0 && !extra_dst) return fail(ONEBIT_ERR_NULL, "null destination list");
  for (int e = 0; e < n_extra; ++e) {
    if (!extra_dst[e]) return fail(ONEBIT_ERR_NULL, "null extra destination %d", e);
    if (reinterpret_cast<uintptr_t>(extra_dst[e]) & 15) return fail(ONEBIT_ERR_ARG, "extra destination %d is not 16-byte aligned", e);
  }
  if (!ob::prefill_scatter_supported(m, n, k, d))
    return fail(ONEBIT_ERR_SHAPE,
                "the multi-destination GEMM needs m %% 256 == 0, k %% 128 == 0, n %% 8 == 0 and a 16-byte aligned d "
                "(got m=%lld n=%lld k=%lld)", (long long)m, (long long)n, (long long)k);
  int* status = nullptr;
  if (int rc = get_status_word(&status)) return rc;
  cudaError_t e = ob::launch_gemm_prefill_scatter(bits_tile, meta_tile, scale, b, d, extra_dst, n_extra, m, n, k, status,
                                                  static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? ONEBIT_OK : cuda_fail(e, "multi-destination GEMM launch");
}

int onebit_sparse_matmul_ex(const void* a_bits, const void* b, void* d, const void* e_meta, const void* scale, int64_t m,
                            int64_t n, int64_t k, int out_type, int meta_dialect, void* workspace, size_t workspace_bytes,
                            void* stream) {
  if (!a_bits || !b || !d || !e_meta) return fail(ONEBIT_ERR_NULL, "null operand pointer");
  if (m <= 0 || n <= 0 || k <= 0 || k % 32 != 0)
    return fail(ONEBIT_ERR_SHAPE, "need m, n > 0 and k %% 32 == 0 (got m=%lld n=%lld k=%lld)", (long long)m, (long long)n, (long long)k);
  if (int rc = check_dialect_rows(meta_dialect, m)) return rc;
  if (out_type != OB_OUT_F32 && out_type != OB_OUT_F16) return fail(ONEBIT_ERR_ARG, "unknown output type %d", out_type);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!tiled_shape(m, k)) {
    cudaError_t e = ob::launch_gemm_simple(a_bits, e_meta, meta_dialect, scale, b, d, m, n, k, out_type, st);
    return e == cudaSuccess ? ONEBIT_OK : cuda_fail(e, "plain GEMM launch");
  }
  const size_t need = onebit_workspace_bytes(m, k);
  const size_t bits_bytes = round256(onebit_packed_bits_bytes(m, k));
  if (workspace) {
    if (workspace_bytes < need) return fail(ONEBIT_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail(ONEBIT_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    void* bits_tile = workspace;
    void* meta_tile = static_cast<char*>(workspace) + bits_bytes;
    cudaError_t e = ob::launch_relayout(a_bits, e_meta, meta_dialect, m, k, bits_tile, meta_tile, st);
    if (e != cudaSuccess) return cuda_fail(e, "relayout launch");
    return matmul_packed_impl(bits_tile, meta_tile, scale, b, d, m, n, k, out_type, ONEBIT_KERNEL_AUTO, st);
  }
  // Library-owned scratch: one block per device, shared by every such call. The whole enqueue happens under
  // the lock and between a wait on and a record of the block's event, so concurrent calls -- other host
  // threads, other streams -- use the block one after the other on the GPU.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cudaError_t e = cudaStreamIsCapturing(st, &cap);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamIsCapturing");
  if (cap != cudaStreamCaptureStatusNone)
    return fail(ONEBIT_ERR_WORKSPACE, "a stream that is being captured needs a caller-provided workspace (the library's own "
                                      "scratch may have to grow, and is ordered by an event outside the capture)");
  int dev = 0;
  if (int rc = current_device(&dev)) return rc;
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  DeviceScratch& s = g_scratch[dev];
  if (int rc = grow_scratch_locked(s, need)) return rc;
  void* bits_tile = s.buf;
  void* meta_tile = static_cast<char*>(s.buf) + bits_bytes;
  e = cudaStreamWaitEvent(st, s.last_use, 0);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent(scratch)");
  e = ob::launch_relayout(a_bits, e_meta, meta_dialect, m, k, bits_tile, meta_tile, st);
  if (e != cudaSuccess) return cuda_fail(e, "relayout launch");
  const int rc = matmul_packed_impl(bits_tile, meta_tile, scale, b, d, m, n, k, out_type, ONEBIT_KERNEL_AUTO, st);
  e = cudaEventRecord(s.last_use, st);   // also after a failed GEMM launch: the relayout already uses the block
  if (rc != ONEBIT_OK) return rc;
  return e == cudaSuccess ? ONEBIT_OK : cuda_fail(e, "cudaEventRecord(scratch)");
}

namespace {
int pack_impl(const void* dense, int dense_dtype, int64_t m, int64_t k, void* sparse, void* a_bits, void* e_meta, int meta_dialect,
              void* bits_tile, void* meta_tile, bool apply_mask, void* masked, void* stream) {
  if (!dense) return fail(ONEBIT_ERR_NULL, "null dense pointer");
  if (dense_dtype < OB_DENSE_F16 || dense_dtype > OB_DENSE_I32) return fail(ONEBIT_ERR_ARG, "unknown dense dtype %d", dense_dtype);
  if (m <= 0 || k <= 0 || k % 32 != 0 || m % 32 != 0)
    return fail(ONEBIT_ERR_SHAPE, "need m %% 32 == 0 and k %% 32 == 0 (got m=%lld k=%lld)", (long long)m, (long long)k);
  if (e_meta) { if (int rc = check_dialect_rows(meta_dialect, m)) return rc; }
  if ((bits_tile || meta_tile) && !tiled_shape(m, k))
    return fail(ONEBIT_ERR_SHAPE, "tile order needs m %% 128 == 0 and k %% 128 == 0 (got m=%lld k=%lld)", (long long)m, (long long)k);
  cudaError_t e = ob::launch_pack(dense, dense_dtype, m, k, sparse, a_bits, e_meta, meta_dialect, bits_tile, meta_tile, apply_mask,
                                  masked, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? ONEBIT_OK : cuda_fail(e, "pack launch");
}
}  // namespace

int onebit_pack_from_dense(const void* dense, int dense_dtype, int64_t m, int64_t k, void* sparse, void* a_bits,
                           void* e_meta, int meta_dialect, void* bits_tile, void* meta_tile, void* stream) {
  return pack_impl(dense, dense_dtype, m, k, sparse, a_bits, e_meta, meta_dialect, bits_tile, meta_tile, false, nullptr, stream);
}

int onebit_mask_pack_from_dense(const void* dense_f16, int64_t m, int64_t k, void* masked_f16, void* sparse, void* a_bits,
                                void* e_meta, int meta_dialect, void* bits_tile, void* meta_tile, void* stream) {
  return pack_impl(dense_f16, OB_DENSE_F16, m, k, sparse, a_bits, e_meta, meta_dialect, bits_tile, meta_tile, true, masked_f16, stream);
}

int onebit_mask24(const void* dense_f16, int64_t count, void* masked_f16, void* mask_u8, void* stream) {
  if (!dense_f16) return fail(ONEBIT_ERR_NULL, "null dense pointer");
  if (count < 0 || count % 8 != 0) return fail(ONEBIT_ERR_SHAPE, "element count %lld must be a multiple of 8", (long long)count);
  cudaError_t e = ob::launch_mask24(dense_f16, count, masked_f16, mask_u8, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? ONEBIT_OK : cuda_fail(e, "mask launch");
}

int onebit_unpack_to_dense(const void* bits_tile, const void* meta_tile, const void* scale, int64_t m, int64_t k,
                           void* dense_f16, void* stream) {
  if (!bits_tile || !meta_tile || !dense_f16) return fail(ONEBIT_ERR_NULL, "null operand pointer");
  if (!tiled_shape(m, k)) return fail(ONEBIT_ERR_SHAPE, "tile order needs m %% 128 == 0 and k %% 128 == 0");
  cudaError_t e = ob::launch_tile_to_dense(bits_tile, meta_tile, scale, m, k, dense_f16, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? ONEBIT_OK : cuda_fail(e, "unpack launch");
}

// Reads and clears the status words of the tensor-memory and decode kernels on the current device. Synchronises
// the device. Returns ONEBIT_ERR_DEVICE_WAIT if a bounded wait inside a kernel gave up since the
// last call.
int onebit_check_device_status(void) {
  int* status = nullptr;
  if (int rc = get_status_word(&status)) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
  int host = 0;
  e = cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(status)");
  if (host != 0) {
    cudaMemset(status, 0, sizeof(int));
    return fail(ONEBIT_ERR_DEVICE_WAIT, "a bounded wait inside the tensor-memory kernel gave up (role code %d)", host);
  }
  e = ob::read_decode_status(&host);
  if (e != cudaSuccess) return cuda_fail(e, "read_decode_status");
  if (host != 0) return fail(ONEBIT_ERR_DEVICE_WAIT, "a bounded wait inside the decode kernel gave up (code %d)", host);
  e = ob::read_fewtok_status(&host);
  if (e != cudaSuccess) return cuda_fail(e, "read_fewtok_status");
  if (host != 0) return fail(ONEBIT_ERR_DEVICE_WAIT, "a bounded wait inside the few-token kernel gave up (code %d)", host);
  return ONEBIT_OK;
}

}  // extern "C"

// The reference's entry point, same C++-mangled symbol (include/onebit_sparse_tensor.h:5 and
// csrc/kernel_lib.cu:23 of the reference).
void onebit_sparse_matmul(void* a, void* b, void* /*c*/, void* d, void* e, int m, int n, int k) {
  onebit_sparse_matmul_ex(a, b, d, e, nullptr, m, n, k, ONEBIT_OUT_F32, ONEBIT_META_CUTLASS, nullptr, 0, nullptr);
}
