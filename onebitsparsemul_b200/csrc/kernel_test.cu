// a.out: the benchmark CLI of the reference (tests/kernel_test.cu, built by `make`), rebuilt on
// libonebitmul. Same flags and the same three output lines (tests/kernel_test.cu:155-177,703-780):
//
//   ./a.out --a_rows=1024 --n=1024 --a_cols=1024 --reference-check=false [--iterations=20]
//     Runtime: <ms> ms
//      GFLOPs: <2*a_rows*n*a_cols / runtime / 1e9>
//     Passed | Failed
//
// --alpha --beta --streams --a_ell_num_columns --a_ell_blocksize --a_base are accepted and ignored
// (alpha = 1, beta = 0 as in csrc/kernel_lib.cu:60-61; the ELL flags were never used). New, optional:
//   --dist=baseline|reference   baseline: random valid 2:4 pattern, Bernoulli signs, tokens N(0,1)
//                               reference: the reference's fill -- all sign bits 1, metadata 0x4444,
//                               tokens uniform integers in [-8, 8] (tests/kernel_test.cu:302-332,398-400)
//   --seed=<int> (3080)  --scale=<bool> per-row fp16 scale U[0.01,0.1]  --out=fp32|fp16
//   --kernel=auto|prefill|decode  --stateless=<bool> time the reference entry point (relayout per call)
//   --json  one JSON object instead of the three lines
//
// The reference check is re-done rather than copied: the reference's is off by default and compares
// a beta = 1 device run with a beta = 0 host run through an uncompress that strides 8 instead of 16
// columns (tests/kernel_test.cu:36-57,449-456,563-575). Here the host recomputes sampled rows (all
// rows when the problem is small) from the same weights with fp32 accumulation: exact match for
// integer tokens, max |err| <= 1e-2 * |row|_inf otherwise.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "onebit_sparse_tensor.h"

#define CK(call)                                                                                   \
  do {                                                                                             \
    cudaError_t e_ = (call);                                                                       \
    if (e_ != cudaSuccess) { fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); return -1; } \
  } while (0)
#define OBCK(call)                                                                                 \
  do {                                                                                             \
    int rc_ = (call);                                                                              \
    if (rc_ != ONEBIT_OK) { fprintf(stderr, "libonebitmul error %d: %s\n", rc_, onebit_last_error()); return -1; } \
  } while (0)

struct Options {
  bool help = false, reference_check = false, scale = false, json = false, stateless = false, fp16_out = false;
  int iterations = 20, a_rows = 1024, n = 1024, a_cols = 1024, kernel = ONEBIT_KERNEL_AUTO;
  unsigned seed = 3080;
  bool dist_reference = false;

  static bool to_bool(const std::string& v) { return !(v == "false" || v == "0" || v == "False"); }
  void parse(int argc, char** argv) {
    for (int i = 1; i < argc; ++i) {
      std::string a = argv[i];
      if (a.rfind("--", 0) != 0) continue;
      a = a.substr(2);
      std::string key = a, val = "true";
      const size_t eq = a.find('=');
      if (eq != std::string::npos) { key = a.substr(0, eq); val = a.substr(eq + 1); }
      if (key == "help") help = true;
      else if (key == "reference-check") reference_check = to_bool(val);
      else if (key == "iterations") iterations = std::max(1, atoi(val.c_str()));
      else if (key == "a_rows") a_rows = atoi(val.c_str());
      else if (key == "n") n = atoi(val.c_str());
      else if (key == "a_cols") a_cols = atoi(val.c_str());
      else if (key == "seed") seed = (unsigned)strtoul(val.c_str(), nullptr, 10);
      else if (key == "scale") scale = to_bool(val);
      else if (key == "json") json = to_bool(val);
      else if (key == "stateless") stateless = to_bool(val);
      else if (key == "out") fp16_out = (val == "fp16");
      else if (key == "dist") dist_reference = (val == "reference");
      else if (key == "kernel") kernel = val == "prefill" ? ONEBIT_KERNEL_PREFILL : val == "decode" ? ONEBIT_KERNEL_DECODE : ONEBIT_KERNEL_AUTO;
      // alpha, beta, streams, a_ell_num_columns, a_ell_blocksize, a_base: accepted, unused
    }
  }
  double gflops(double runtime_s) const { return 2.0 * double(a_rows) * double(a_cols) * double(n) / 1.0e9 / runtime_s; }
};

static void usage() {
  printf("1 Bit Sparse _gemm\n\n  Profiles the one-bit 2:4 sparse GEMM kernels of libonebitmul.\n\nOptions:\n\n"
         "  --help                      If specified, displays this usage statement.\n\n"
         "  --a_rows=<int>              Sets the number of the rows of the sparse matrix.\n"
         "  --n=<int>                   Sets the N dimension.\n"
         "  --a_cols=<int>              Sets the number of columns of the sparse matrix.\n"
         "  --iterations=<int>          Number of profiling iterations to perform.\n"
         "  --reference-check=<bool>    If true, performs reference check.\n"
         "  --dist=baseline|reference   Input distributions (see the head of this file).\n"
         "  --seed=<int> --scale=<bool> --out=fp32|fp16 --kernel=auto|prefill|decode --stateless=<bool> --json\n"
         "  --alpha --beta --streams --a_ell_num_columns --a_ell_blocksize --a_base   accepted, ignored\n");
}

// ---- counter-based generators, identical on host and device ------------------------------------------
__host__ __device__ inline uint32_t mix32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
  return (uint32_t)x;
}
__host__ __device__ inline uint32_t rnd(unsigned seed, unsigned stream, uint64_t idx) {
  return mix32(((uint64_t)seed << 40) ^ ((uint64_t)stream << 36) ^ idx);
}

// dense fp16 weights: one valid 2:4 pattern and two signs per group of 4
__global__ void fill_weights(__half* w, int64_t groups, unsigned seed) {
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  const uint32_t r = rnd(seed, 1, (uint64_t)g);
  const unsigned nibs[6] = {0x4, 0x8, 0x9, 0xC, 0xD, 0xE};
  const unsigned nib = nibs[r % 6];
  const int i0 = nib & 3, i1 = nib >> 2;
  __half v[4] = {__float2half(0.f), __float2half(0.f), __float2half(0.f), __float2half(0.f)};
  v[i0] = __float2half((r >> 8) & 1 ? 1.f : -1.f);
  v[i1] = __float2half((r >> 9) & 1 ? 1.f : -1.f);
  *reinterpret_cast<uint2*>(w + g * 4) = *reinterpret_cast<uint2*>(v);
}
__global__ void fill_tokens(__half* b, int64_t count, unsigned seed, int integer) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const uint32_t r1 = rnd(seed, 2, (uint64_t)i), r2 = rnd(seed, 3, (uint64_t)i);
  float v;
  if (integer) v = (float)((int)(r1 % 17) - 8);
  else {
    const float u1 = (r1 + 1.0f) * (1.0f / 4294967808.0f), u2 = r2 * (1.0f / 4294967296.0f);
    v = sqrtf(-2.f * logf(u1)) * cosf(6.2831853f * u2);
  }
  b[i] = __float2half(v);
}
__global__ void fill_scale(__half* s, int64_t count, unsigned seed) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) s[i] = __float2half(0.01f + 0.09f * (rnd(seed, 4, (uint64_t)i) * (1.0f / 4294967296.0f)));
}

int main(int argc, char** argv) {
  Options o;
  o.parse(argc, argv);
  if (o.help) { usage(); return 0; }
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { fprintf(stderr, "no CUDA device: this program has no CPU path\n"); return -1; }
  cudaDeviceProp prop;
  CK(cudaGetDeviceProperties(&prop, 0));
  if (prop.major < 10) { fprintf(stderr, "libonebitmul is built for sm_100a; found compute capability %d.%d\n", prop.major, prop.minor); return -1; }

  const int64_t m = o.a_rows, n = o.n, k = o.a_cols;
  if (m % 128 != 0 || k % 128 != 0 || n < 1) { fprintf(stderr, "a_rows and a_cols must be multiples of 128, n >= 1\n"); return -1; }
  const bool integer_tokens = o.dist_reference;

  __half *d_w = nullptr, *d_b = nullptr, *d_scale = nullptr;
  void *d_bits_ref = nullptr, *d_meta_ref = nullptr, *d_bits_tile = nullptr, *d_meta_tile = nullptr, *d_out = nullptr;
  const size_t out_elem = o.fp16_out ? 2 : 4;
  CK(cudaMalloc(&d_b, (size_t)k * n * 2));
  CK(cudaMalloc(&d_out, (size_t)m * n * out_elem));
  CK(cudaMalloc(&d_bits_ref, (size_t)m * k / 16));
  CK(cudaMalloc(&d_meta_ref, (size_t)m * k / 8));
  CK(cudaMalloc(&d_bits_tile, onebit_packed_bits_bytes(m, k)));
  CK(cudaMalloc(&d_meta_tile, onebit_packed_meta_bytes(m, k)));
  CK(cudaMalloc(&d_w, (size_t)m * k * 2));
  if (o.scale) { CK(cudaMalloc(&d_scale, (size_t)m * 2)); fill_scale<<<(unsigned)((m + 255) / 256), 256>>>(d_scale, m, o.seed); }
  fill_tokens<<<(unsigned)((k * n + 255) / 256), 256>>>(d_b, k * n, o.seed, integer_tokens);
  if (o.dist_reference) {
    // all sign bits 1, metadata 0x4444: W keeps dense columns 4g and 4g+1 with +1
    CK(cudaMemset(d_bits_ref, 0xFF, (size_t)m * k / 16));
    std::vector<uint16_t> e((size_t)m * k / 16, 0x4444);
    CK(cudaMemcpy(d_meta_ref, e.data(), e.size() * 2, cudaMemcpyHostToDevice));
    OBCK(onebit_relayout(d_bits_ref, d_meta_ref, ONEBIT_META_CUTLASS, m, k, d_bits_tile, d_meta_tile, nullptr));
    std::vector<__half> w((size_t)m * k);
    for (size_t i = 0; i < w.size(); ++i) w[i] = __float2half((i % 4) < 2 ? 1.f : 0.f);
    CK(cudaMemcpy(d_w, w.data(), w.size() * 2, cudaMemcpyHostToDevice));
  } else {
    fill_weights<<<(unsigned)((m * k / 4 + 255) / 256), 256>>>(d_w, m * k / 4, o.seed);
    OBCK(onebit_pack_from_dense(d_w, ONEBIT_DENSE_F16, m, k, nullptr, d_bits_ref, d_meta_ref, ONEBIT_META_CUTLASS,
                                d_bits_tile, d_meta_tile, nullptr));
  }
  CK(cudaDeviceSynchronize());

  auto run = [&]() -> int {
    if (o.stateless) {
      if (o.fp16_out || o.scale)
        return onebit_sparse_matmul_ex(d_bits_ref, d_b, d_out, d_meta_ref, d_scale, m, n, k, o.fp16_out ? ONEBIT_OUT_F16 : ONEBIT_OUT_F32,
                                       ONEBIT_META_CUTLASS, nullptr, 0, nullptr);
      onebit_sparse_matmul(d_bits_ref, d_b, d_out, d_out, d_meta_ref, (int)m, (int)n, (int)k);
      return ONEBIT_OK;
    }
    return onebit_matmul_packed(d_bits_tile, d_meta_tile, d_scale, d_b, d_out, m, n, k, o.fp16_out ? ONEBIT_OUT_F16 : ONEBIT_OUT_F32,
                                o.kernel, nullptr);
  };

  OBCK(run());                         // first run + warm-up, as the reference does
  CK(cudaDeviceSynchronize());
  OBCK(onebit_check_device_status());

  bool passed = true;
  double worst = 0.0;
  if (o.reference_check) {
    // host check on sampled rows: W rows and B copied back, fp32 accumulation in increasing k
    const int64_t max_rows = ((double)m * n * k <= 4.0e9) ? m : 64;
    std::vector<__half> hb((size_t)k * n), hw((size_t)k), hs(m);
    CK(cudaMemcpy(hb.data(), d_b, hb.size() * 2, cudaMemcpyDeviceToHost));
    if (o.scale) CK(cudaMemcpy(hs.data(), d_scale, (size_t)m * 2, cudaMemcpyDeviceToHost));
    std::vector<float> bf((size_t)k * n), acc(n);
    for (size_t i = 0; i < bf.size(); ++i) bf[i] = __half2float(hb[i]);
    std::vector<char> row_out((size_t)n * out_elem);
    for (int64_t s = 0; s < max_rows && passed; ++s) {
      const int64_t i = (max_rows == m) ? s : (int64_t)(rnd(o.seed, 5, (uint64_t)s) % (uint32_t)m);
      CK(cudaMemcpy(hw.data(), d_w + i * k, (size_t)k * 2, cudaMemcpyDeviceToHost));
      CK(cudaMemcpy(row_out.data(), (char*)d_out + (size_t)i * n * out_elem, row_out.size(), cudaMemcpyDeviceToHost));
      std::fill(acc.begin(), acc.end(), 0.f);
      for (int64_t kk = 0; kk < k; ++kk) {
        const float w = __half2float(hw[kk]);
        if (w == 0.f) continue;
        const float* br = &bf[(size_t)kk * n];
        if (w > 0) for (int64_t j = 0; j < n; ++j) acc[j] += br[j];
        else for (int64_t j = 0; j < n; ++j) acc[j] -= br[j];
      }
      const float sc = o.scale ? __half2float(hs[i]) : 1.f;
      float rowmax = 0.f, err = 0.f;
      for (int64_t j = 0; j < n; ++j) {
        const float want = acc[j] * sc;
        const float got = o.fp16_out ? __half2float(reinterpret_cast<__half*>(row_out.data())[j]) : reinterpret_cast<float*>(row_out.data())[j];
        rowmax = std::max(rowmax, std::fabs(want));
        err = std::max(err, std::fabs(got - want));
        if (std::isnan(got)) err = INFINITY;
      }
      const bool exact_expected = integer_tokens && !o.scale && !o.fp16_out;
      if (exact_expected ? (err != 0.f) : (err > 1e-2f * rowmax)) passed = false;
      worst = std::max(worst, (double)(rowmax > 0 ? err / rowmax : err));
    }
  }

  cudaEvent_t ev0, ev1;
  CK(cudaEventCreate(&ev0));
  CK(cudaEventCreate(&ev1));
  CK(cudaEventRecord(ev0));
  for (int it = 0; it < o.iterations; ++it) OBCK(run());
  CK(cudaEventRecord(ev1));
  CK(cudaEventSynchronize(ev1));
  OBCK(onebit_check_device_status());
  float ms = 0.f;
  CK(cudaEventElapsedTime(&ms, ev0, ev1));
  const double runtime_ms = double(ms) / o.iterations;
  const double gflops = o.gflops(runtime_ms / 1000.0);

  if (o.json) {
    printf("{\"a_rows\": %lld, \"n\": %lld, \"a_cols\": %lld, \"runtime_ms\": %.6f, \"gflops\": %.3f, \"iterations\": %d, "
           "\"checked\": %s, \"passed\": %s, \"worst_rel_err\": %.3e, \"path\": \"%s\"}\n",
           (long long)m, (long long)n, (long long)k, runtime_ms, gflops, o.iterations, o.reference_check ? "true" : "false",
           passed ? "true" : "false", worst, o.stateless ? "stateless" : "prepacked");
  } else {
    printf("Runtime: %g ms\n", runtime_ms);
    printf(" GFLOPs: %g\n", gflops);
    printf(passed ? "Passed\n" : "Failed\n");
  }
  return passed ? 0 : -1;
}
