/*
 * libonebitmul -- C = A_sparse x B on NVIDIA B200 (sm_100a).
 *   A : one-bit (+-1) 2:4 structured-sparse weight matrix, m x k, 1.5 bit per dense weight,
 *       optional per-row fp16 scale
 *   B : dense fp16 activations, k x n row-major (n contiguous)
 *   C : m x n row-major, fp32 or fp16, fp32 accumulation
 *
 * This header is the drop-in boundary for the reference's include/onebit_sparse_tensor.h. The first
 * declaration keeps the reference's exact signature and C++ linkage; everything inside extern "C"
 * is additive. All pointers are DEVICE pointers on the current device unless stated otherwise.
 * Nothing here synchronises the device; work is queued on the given stream (the legacy entry point
 * uses the default stream, as the reference does).
 *
 * Operand orders
 *   "reference order": what the reference's kernel and Python packer exchange --
 *        sign bits  uint8 (k/2, m/8): bit (i & 7) of byte [q][i >> 3] is kept value q of row i
 *                   (1 = +1, 0 = -1), i.e. a column-major-in-m 1-bit matrix (csrc/kernel.h:13-15)
 *        metadata   uint16 (m, k/16) in one of two shuffles (ONEBIT_META_*), 4 nibbles per word,
 *                   nibble = idx0 | idx1 << 2 of the two kept positions of a group of 4
 *   "tile order": this library's own streaming order (one 1 KiB sign block and one 2 KiB metadata
 *        block per 128 x 128 tile; see onebit_packed_*_bytes). Produced by onebit_relayout or
 *        onebit_pack_from_dense, consumed by onebit_matmul_packed. Needs m % 128 == 0, k % 128 == 0.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

/* Replaces include/onebit_sparse_tensor.h:5 of the reference (defined in csrc/kernel_lib.cu:23-97),
 * same symbol (_Z20onebit_sparse_matmulPvS_S_S_S_iii):
 *   a  sign bits, reference order          b  fp16 (k, n)
 *   c  ignored (beta = 0; may alias d)     d  fp32 (m, n) output
 *   e  metadata, ONEBIT_META_CUTLASS order (what the reference kernel's E operand is)
 * Runs on the default stream. Where the reference prints and exit()s on error, this records the
 * error for onebit_last_error() and returns without launching. */
#ifdef __cplusplus
void onebit_sparse_matmul(void *a, void *b, void *c, void *d, void *e, int m, int n, int k);
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum { ONEBIT_META_PYTHON = 0,   /* onebit_sparse_mul/_semi_structured_conversions.py:21-48 */
       ONEBIT_META_CUTLASS = 1 };/* CUTLASS reorder_meta + ColumnMajorInterleaved<2> (csrc/threadblock.h:198-199) */
enum { ONEBIT_OUT_F32 = 0, ONEBIT_OUT_F16 = 1 };
enum { ONEBIT_DENSE_F16 = 0, ONEBIT_DENSE_BF16 = 1, ONEBIT_DENSE_I32 = 2 };
enum { ONEBIT_KERNEL_AUTO = 0,    /* few-token kernel for n <= 16 (n <= 32 up to 8192 rows) or n % 8 != 0, tile kernels otherwise */
       ONEBIT_KERNEL_PREFILL = 1, /* TMA + tcgen05.mma.sp kernel */
       ONEBIT_KERNEL_DECODE = 2,  /* split-K cluster kernel for few tokens */
       /* Flag, OR-ed into any of the above: the caller vouches that the packed weights of this call were
        * complete before the kernel that precedes this call in `stream` was launched (weights packed at load
        * time, as in a decode loop). The few-token kernel then requests them while that kernel still drains.
        * Without the flag it requests nothing before that kernel has completed and its writes are visible. */
       ONEBIT_KERNEL_STABLE_WEIGHTS = 0x100 };

enum { ONEBIT_OK = 0, ONEBIT_ERR_SHAPE = 1, ONEBIT_ERR_NULL = 2, ONEBIT_ERR_CUDA = 3,
       ONEBIT_ERR_WORKSPACE = 4, ONEBIT_ERR_ARG = 5, ONEBIT_ERR_DEVICE_WAIT = 6 };

/* Message of the calling thread's most recent failed call ("" if none). Host pointer, valid until
 * the thread's next failing call. Replaces the reference's exit(EXIT_FAILURE) (csrc/kernel_lib.cu:11-20). */
const char *onebit_last_error(void);

/* Bytes of the tile-ordered operands of an m x k matrix (m, k multiples of 128):
 * m*k/16 and m*k/8. */
size_t onebit_packed_bits_bytes(int64_t m, int64_t k);
size_t onebit_packed_meta_bytes(int64_t m, int64_t k);
/* Scratch bytes onebit_sparse_matmul_ex needs for a call of this shape (the two above, each
 * rounded up to 256). */
size_t onebit_workspace_bytes(int64_t m, int64_t k);

/* Stateless GEMM on reference-ordered operands: the generalisation of onebit_sparse_matmul
 * (csrc/kernel_lib.cu:23-97) by a per-row scale (NULL = none), an fp16 output, a choice of metadata
 * order and a stream. Internally: relayout into `workspace`, then the dispatched kernel.
 * workspace == NULL makes the library use one cached block per device, grown by cudaMalloc on demand
 * and never freed while the process lives. Calls that share the block are ordered on the GPU by an
 * event (each call's relayout waits for the previous call's GEMM), from whatever host threads and
 * streams they come, so they are safe but do not overlap; pass per-stream workspaces for concurrency.
 * Not usable on a stream that is being captured (ONEBIT_ERR_WORKSPACE): pass a workspace there.
 * Shapes the tiled kernels do not take
 * (m % 128, k % 128 != 0; needs m % 32 == 0 (64 for ONEBIT_META_PYTHON), k % 32 == 0) run on a plain
 * CUDA-core kernel without workspace. stream is a cudaStream_t. */
int onebit_sparse_matmul_ex(const void *a_bits, const void *b, void *d, const void *e_meta, const void *scale,
                            int64_t m, int64_t n, int64_t k, int out_type, int meta_dialect,
                            void *workspace, size_t workspace_bytes, void *stream);

/* Reference order -> tile order; the once-per-weight half of onebit_sparse_matmul_ex. It is the
 * device-side counterpart of handing pack()'s tensors (onebit_sparse_mul/__init__.py:130-145) to
 * the kernel. All four buffers must be 16-byte aligned (so must a_bits and e_meta of the stateless entry
 * points; the reference's kernel asks the same of its A and E operands, csrc/kernel.h:19-21). */
int onebit_relayout(const void *a_bits, const void *e_meta, int meta_dialect, int64_t m, int64_t k,
                    void *bits_tile, void *meta_tile, void *stream);

/* GEMM on tile-ordered operands (the fast path; the hot loop of BinaryLinear_2_4.forward,
 * onebit_sparse_mul/__init__.py:118-128). kernel: ONEBIT_KERNEL_*.
 * The few-token kernel is launched with programmatic stream serialisation: its grid may start while the
 * kernel before it in `stream` drains. By default it touches no operand before that kernel has completed
 * (a producer such as onebit_relayout or onebit_pack_from_dense may sit directly before it). With
 * ONEBIT_KERNEL_STABLE_WEIGHTS it requests the packed weights first and waits only then; tokens are read,
 * and d is written, after the wait in either case. Set ONEBIT_PDL=0 in the environment to launch it as an
 * ordinary kernel. */
int onebit_matmul_packed(const void *bits_tile, const void *meta_tile, const void *scale, const void *b, void *d,
                         int64_t m, int64_t n, int64_t k, int out_type, int kernel, void *stream);

/* onebit_matmul_packed with fp16 output written to SEVERAL buffers in one pass: d (m, n) and n_extra <= 7
 * more buffers of the same shape and row stride n, given as a HOST array of device-accessible pointers
 * (16-byte aligned). Meant for a GEMM sharded by rows of A over the GPUs of one node whose full result
 * every GPU needs: each GPU passes, as extra destinations, the addresses of its row slab inside the peers'
 * copies of C (peer-mapped memory), and the epilogue's stores cross NVLink while the next tile is being
 * multiplied -- the all-gather is fused into the GEMM. The caller orders the GPUs before and after
 * (a barrier before peers may be overwritten, one before they are read). Needs m % 256 == 0, k % 128 == 0,
 * n % 8 == 0. No counterpart in the reference, which is single-GPU (csrc/kernel_lib.cu:23-97). */
int onebit_matmul_packed_scatter(const void *bits_tile, const void *meta_tile, const void *scale, const void *b, void *d,
                                 void *const *extra_dst, int n_extra, int64_t m, int64_t n, int64_t k, void *stream);

/* The same product in the nn.Linear convention, for callers that keep activations token-major:
 *   y (n, m) = x (n, k) @ W^T (+ bias),  x fp16 row-major, y fp16 / fp32 row-major, bias fp16 (m) or NULL,
 * W given by its tile-ordered operands and optional per-row scale. It is C^T = (A_sparse x B)^T with
 * B = x^T, computed without any transposition pass: x is loaded as a K-major tensor-core operand and
 * the epilogue writes the transposed tile. This is what the reference's model-replace demo needs
 * (tests/python/test_model_replace.py:22-44; its forward passes x straight through,
 * onebit_sparse_mul/__init__.py:118-128). n <= 16 runs on the split-K cluster kernel, more tokens on
 * the CTA-pair tensor-memory kernel (needs m % 256 == 0; otherwise the cluster kernel serves any n).
 * x must be 16-byte aligned. kernel: ONEBIT_KERNEL_* (ONEBIT_KERNEL_STABLE_WEIGHTS as above). */
int onebit_linear_tokens(const void *bits_tile, const void *meta_tile, const void *scale, const void *bias, const void *x,
                         void *y, int64_t m, int64_t n, int64_t k, int out_type, int kernel, void *stream);

/* The same GEMM for tokens and results that live in (pinned) HOST memory: b_host fp16 (k, n) and d_host
 * (m, n), both row-major. The reference's Python wrapper hands the kernel a CPU-allocated C
 * (onebit_sparse_mul/__init__.py:12-15); here the transfers are part of the call and overlap the
 * compute: token column panels go host -> device, are multiplied and return device -> host in a
 * three-slot pipeline on internal streams, so a call costs about max(H2D, D2H). `workspace` is DEVICE
 * memory of onebit_host_workspace_bytes(m, n, k, out_type) bytes, 256-byte aligned, owned by the caller
 * and busy until the work queued by this call has finished. Asynchronous like the other calls: work
 * queued on `stream` before the call precedes it, work queued after it follows it. Calls on one device
 * share three internal streams: a call is enqueued as a whole under a lock, and a later call's legs queue
 * behind the earlier call's on those streams, so concurrent callers are safe and serialise. Each call
 * that may overlap another needs its own workspace. Needs n % 8 == 0. */
size_t onebit_host_workspace_bytes(int64_t m, int64_t n, int64_t k, int out_type);
int onebit_matmul_packed_host(const void *bits_tile, const void *meta_tile, const void *scale, const void *b_host,
                              void *d_host, int64_t m, int64_t n, int64_t k, int out_type, void *workspace,
                              size_t workspace_bytes, void *stream);

/* Pitched asynchronous copy between host and device (either direction, decided by the pointers): `rows` rows of
 * `row_bytes` bytes, `dst_pitch` / `src_pitch` bytes from one row to the next. The building block of the
 * host-buffer paths -- a column panel of a row-major matrix is such a block -- exported for callers that
 * pipeline panels themselves (the row-sharded host path of onebitsparsemul_b200/sharded.py). Host memory must be
 * page-locked for the copy to be asynchronous. No counterpart in the reference. */
int onebit_copy_2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t row_bytes,
                         size_t rows, void *stream);

/* Dense (m, k) row-major weights -> packed operands in one pass; bit-exact replacement of
 * sparse_semi_structured_from_dense_cutlass + binary_quant + .T + pack_binary
 * (_semi_structured_conversions.py:54-179, onebit_sparse_mul/__init__.py:22-34,139-143).
 * Every output pointer may be NULL (not produced):
 *   sparse     (m, k/2) kept values, dense dtype     a_bits   sign bits, reference order
 *   e_meta     metadata in meta_dialect order        bits_tile / meta_tile   tile order
 * The input is expected to be 2:4 already; other groups follow the reference's encoder table
 * (_semi_structured_conversions.py:99-124). Needs k % 32 == 0 and m % 32 == 0 (m % 64 == 0 for
 * ONEBIT_META_PYTHON, as the reference's scatter does); tile outputs need m, k % 128 == 0. */
int onebit_pack_from_dense(const void *dense, int dense_dtype, int64_t m, int64_t k, void *sparse,
                           void *a_bits, void *e_meta, int meta_dialect, void *bits_tile, void *meta_tile,
                           void *stream);

/* The whole of BinaryLinear_2_4.pack (onebit_sparse_mul/__init__.py:130-145) in ONE pass over unmasked fp16
 * weights: mask_creator (_semi_structured_conversions.py:286-314; tie rule as onebit_mask24) applied in registers,
 * then everything onebit_pack_from_dense does. Bit-exact with onebit_mask24 followed by onebit_pack_from_dense,
 * without writing and re-reading the masked copy; masked_f16 (m, k) receives that copy only if it is not NULL.
 * Same shape rules and nullable outputs as onebit_pack_from_dense. */
int onebit_mask_pack_from_dense(const void *dense_f16, int64_t m, int64_t k, void *masked_f16, void *sparse, void *a_bits,
                                void *e_meta, int meta_dialect, void *bits_tile, void *meta_tile, void *stream);

/* Magnitude 2:4 mask of fp16 weights (mask_creator, _semi_structured_conversions.py:286-314): in
 * every group of 4 the two smallest |w| are dropped; among equal magnitudes the lower index is
 * dropped first. masked (fp16, same shape) and mask (uint8 0/1) may each be NULL. count % 8 == 0. */
int onebit_mask24(const void *dense_f16, int64_t count, void *masked_f16, void *mask_u8, void *stream);

/* Tile order -> dense fp16 (m, k) holding {-1, 0, +1} * scale (scale NULL = 1): the inverse of the
 * pack (sparse_semi_structured_to_dense_cutlass + dequant_desparse_tile,
 * _semi_structured_conversions.py:186-283, onebit_sparse_mul/__init__.py:47-65). */
int onebit_unpack_to_dense(const void *bits_tile, const void *meta_tile, const void *scale, int64_t m, int64_t k,
                           void *dense_f16, void *stream);

/* The stateless GEMM for callers that cannot allocate device memory -- a server whose own pool owns
 * the whole GPU, a decode loop that cannot take cudaMalloc's device-wide synchronisation, a host that
 * forbids allocation after start-up. No counterpart in the reference (its entry point allocates a
 * CUTLASS workspace object per call, csrc/kernel_lib.cu:73-76). Same operands as
 * onebit_sparse_matmul_ex, but the tile-ordered copy of the weights goes into a fixed array inside
 * the library image (held by every GPU that loads the library, until exit) instead of a workspace:
 *   - m * k <= ONEBIT_STATIC_MAX_WEIGHTS, m % 128 == 0, k % 128 == 0, else an error and no launch;
 *   - always the split-K cluster kernel (meant for few tokens; any n works);
 *   - the first call per device looks up the array's device address, and with CUDA's lazy module loading
 *     that look-up is also the moment the driver loads this part of the library and reserves the array
 *     (about 8 MiB): make one warm-up call per device at start-up, outside stream capture, while device
 *     memory is still available. Later calls touch no allocator;
 *   - calls share the array: two calls that overlap on the GPU race -- serialise them;
 *   - calls no cudaMalloc / cudaFree or allocating library routine. */
#define ONEBIT_STATIC_MAX_WEIGHTS (4096LL * 11008LL)
int onebit_sparse_matmul_static(const void *a_bits, const void *b, void *d, const void *e_meta, const void *scale,
                                int64_t m, int64_t n, int64_t k, int out_type, int meta_dialect, void *stream);

/* Synchronises the current device, then reads and clears its status word: ONEBIT_ERR_DEVICE_WAIT if
 * a bounded wait inside the tensor-memory kernel gave up since the last call (the kernel then still
 * terminated, with an unusable result), ONEBIT_OK otherwise. The reference has no counterpart; its
 * kernel has no device-side waits on other agents. */
int onebit_check_device_status(void);

#ifdef __cplusplus
}
#endif
