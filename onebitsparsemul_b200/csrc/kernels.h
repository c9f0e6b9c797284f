// Launchers of the CUDA kernels behind the C ABI (internal header).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ob {

// Multiprocessors of the current device (cached per device; the dispatchers size their grids by it).
int sm_count();

// K1 (pack.cu)
// apply_mask (fp16 only): the 2:4 magnitude mask is applied in the same pass; masked (nullable) receives the masked weights
cudaError_t launch_pack(const void* dense, int dense_dtype, int64_t m, int64_t k, void* sparse,
                        void* bits_ref, void* meta_ref, int dialect, void* bits_tile, void* meta_tile,
                        bool apply_mask, void* masked, cudaStream_t stream);
// 2:4 magnitude mask (mask.cu)
cudaError_t launch_mask24(const void* dense_f16, int64_t count, void* masked_f16, void* mask_u8,
                          cudaStream_t stream);
// K4 (relayout.cu)
cudaError_t launch_relayout(const void* bits_ref, const void* meta_ref, int dialect, int64_t m, int64_t k,
                            void* bits_tile, void* meta_tile, cudaStream_t stream);
cudaError_t launch_tile_to_dense(const void* bits_tile, const void* meta_tile, const void* scale, int64_t m,
                                 int64_t k, void* dense, cudaStream_t stream);
// plain one-thread-per-output kernel on the reference orders (gemm_simple.cu)
cudaError_t launch_gemm_simple(const void* bits_ref, const void* meta_ref, int dialect, const void* scale,
                               const void* b, void* d, int64_t m, int64_t n, int64_t k, int out_type,
                               cudaStream_t stream);
// K3: decode kernel, n small (gemm_decode.cu). tile-ordered operands. fresh_weights: the weight buffers were
// written by the kernel launched just before on the same stream (the kernel then loads nothing before that one is done).
cudaError_t launch_gemm_decode(const void* bits_tile, const void* meta_tile, const void* scale, const void* b,
                               void* d, int64_t m, int64_t n, int64_t k, int out_type, bool fresh_weights,
                               cudaStream_t stream);
// K2: tcgen05 kernel (gemm_prefill_sm100.cu). tile-ordered operands; n % 8 == 0.
// status: device word that receives a non-zero code if a bounded wait inside the kernel gave up.
cudaError_t launch_gemm_prefill(const void* bits_tile, const void* meta_tile, const void* scale, const void* b,
                                void* d, int64_t m, int64_t n, int64_t k, int out_type, int* status,
                                cudaStream_t stream);
bool prefill_supported(int64_t m, int64_t n, int64_t k);
// token-major forms (x (n, k), y (n, m), optional bias (m)): the nn.Linear convention
cudaError_t launch_gemm_prefill_tokens(const void* bits_tile, const void* meta_tile, const void* scale, const void* bias,
                                       const void* x, void* y, int64_t m, int64_t n, int64_t k, int out_type, int* status,
                                       cudaStream_t stream);
bool prefill_tokens_supported(int64_t m, int64_t n, int64_t k);
// K2 persistent pair kernel with several destinations: the fp16 result goes to d and to n_extra (<= 7) more
// buffers of the same shape (any address this device can store to, e.g. peer GPUs' memory).
cudaError_t launch_gemm_prefill_scatter(const void* bits_tile, const void* meta_tile, const void* scale, const void* b,
                                        void* d, void* const* extra_dst, int n_extra, int64_t m, int64_t n, int64_t k,
                                        int* status, cudaStream_t stream);
bool prefill_scatter_supported(int64_t m, int64_t n, int64_t k, const void* d);
cudaError_t launch_gemm_decode_tokens(const void* bits_tile, const void* meta_tile, const void* scale, const void* bias,
                                      const void* x, void* y, int64_t m, int64_t n, int64_t k, int out_type,
                                      bool fresh_weights, cudaStream_t stream);
// Reads and clears the decode kernel's bounded-wait status on the current device (0 = nothing gave up).
cudaError_t read_decode_status(int* out);
// K3, tensor-memory form (gemm_decode_sm100.cu): the few-token kernel on tcgen05.mma.sp with a 128 x 16 accumulator.
// Same operands as the two launchers above; token_major selects x (n, k) / y (n, m).
cudaError_t launch_gemm_fewtok(const void* bits_tile, const void* meta_tile, const void* scale, const void* bias,
                               const void* b, void* d, int64_t m, int64_t n, int64_t k, int out_type, bool token_major,
                               bool fresh_weights, cudaStream_t stream);
cudaError_t read_fewtok_status(int* out);

}  // namespace ob
