// Times the reference's own host check GEMM on the CPU: the exact template instantiation its benchmark CLI uses
// for --reference-check (tests/kernel_test.cu:441-456 of the reference),
//   cutlass::reference::host::Gemm<half, ColumnMajor, half, RowMajor, float, RowMajor, float, float>,
// from the CUTLASS headers found on this machine (CUTLASS is an un-vendored submodule of the reference; its pinned
// commit is unknown). TEST / BASELINE INFRASTRUCTURE: built into oracle/_ref/ by oracle/build_ref.py, run by the
// benchmark as a reported baseline and by a test that pins the oracle against it; never linked into the library.
//
//   ref_host_gemm <m> <n> <k> [seed]      prints: seconds gflops checksum
//
// A is a dense {-1, 0, +1} matrix with a random valid 2:4 pattern (what the reference's convert + uncompress
// steps, tests/kernel_test.cu:81-117 and :24-59, are meant to produce), B holds integers in [-8, 8] (the
// reference's fill, tests/kernel_test.cu:321-332), so every sum is exact and the checksum is reproducible.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "cutlass/cutlass.h"
#include "cutlass/gemm/gemm.h"
#include "cutlass/layout/matrix.h"
#include "cutlass/numeric_types.h"
#include "cutlass/tensor_ref.h"
#include "cutlass/util/reference/host/gemm.h"

static uint64_t next(uint64_t& s) {            // splitmix64
  uint64_t z = (s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

int main(int argc, char** argv) {
  if (argc < 4) { std::fprintf(stderr, "usage: %s m n k [seed]\n", argv[0]); return 2; }
  const int m = std::atoi(argv[1]), n = std::atoi(argv[2]), k = std::atoi(argv[3]);
  uint64_t seed = argc > 4 ? std::strtoull(argv[4], nullptr, 10) : 3080;
  using half = cutlass::half_t;
  std::vector<half> A((size_t)m * k), B((size_t)k * n);
  std::vector<float> C((size_t)m * n, 0.f), D((size_t)m * n, 0.f);
  static const int pairs[6][2] = {{0, 1}, {0, 2}, {1, 2}, {0, 3}, {1, 3}, {2, 3}};
  for (int i = 0; i < m; ++i)
    for (int g = 0; g < k / 4; ++g) {
      const uint64_t r = next(seed);
      const int* p = pairs[r % 6];
      for (int t = 0; t < 4; ++t) A[(size_t)(4 * g + t) * m + i] = half(0.f);            // column-major: (row i, col c) at c*m + i
      A[(size_t)(4 * g + p[0]) * m + i] = half(((r >> 8) & 1) ? 1.f : -1.f);
      A[(size_t)(4 * g + p[1]) * m + i] = half(((r >> 9) & 1) ? 1.f : -1.f);
    }
  for (size_t i = 0; i < B.size(); ++i) B[i] = half((float)((int)(next(seed) % 17) - 8));
  cutlass::TensorRef<half, cutlass::layout::ColumnMajor> a(A.data(), cutlass::layout::ColumnMajor(m));
  cutlass::TensorRef<half, cutlass::layout::RowMajor> b(B.data(), cutlass::layout::RowMajor(n));
  cutlass::TensorRef<float, cutlass::layout::RowMajor> c(C.data(), cutlass::layout::RowMajor(n)), d(D.data(), cutlass::layout::RowMajor(n));
  cutlass::reference::host::Gemm<half, cutlass::layout::ColumnMajor, half, cutlass::layout::RowMajor, float,
                                 cutlass::layout::RowMajor, float, float> gemm;
  const auto t0 = std::chrono::steady_clock::now();
  gemm({m, n, k}, 1.f, a, b, 0.f, c, d, 0.f);
  const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  double sum = 0;
  for (size_t i = 0; i < D.size(); ++i) sum += D[i] * (double)((i % 7) + 1);
  std::printf("%.6f %.4f %.1f\n", s, 2.0 * m * n * k / s / 1e9, sum);
  return 0;
}
