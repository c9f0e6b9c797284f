// Link smoke test of libonebitmul (the role of the reference's tests/libso_test.cu): links against
// the shared library and calls the reference entry point on a real, tiny problem instead of
// uninitialised pointers.
#include <cuda_runtime.h>

#include <cstdio>
#include <vector>

#include "onebit_sparse_tensor.h"

int main() {
  const int m = 128, n = 8, k = 128;
  void *a, *b, *d, *e;
  if (cudaMalloc(&a, m * k / 16) != cudaSuccess) { printf("no CUDA device\n"); return 1; }
  cudaMalloc(&b, k * n * 2);
  cudaMalloc(&d, m * n * 4);
  cudaMalloc(&e, m * k / 8);
  cudaMemset(a, 0xFF, m * k / 16);                       // all signs +1
  std::vector<unsigned short> meta(m * k / 16, 0x4444), tokens(k * n, 0x3C00 /* 1.0 */);
  cudaMemcpy(e, meta.data(), meta.size() * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(b, tokens.data(), tokens.size() * 2, cudaMemcpyHostToDevice);
  onebit_sparse_matmul(a, b, d, d, e, m, n, k);
  std::vector<float> out(m * n);
  cudaMemcpy(out.data(), d, out.size() * 4, cudaMemcpyDeviceToHost);
  if (onebit_check_device_status() != ONEBIT_OK) { printf("%s\n", onebit_last_error()); return 1; }
  for (float v : out) if (v != float(k / 2)) { printf("Failed: %f\n", v); return 1; }
  printf("Passed\n");
  return 0;
}
