// torch extension module `onebit_sparse_cuda`: the binding the reference builds from
// onebit_sparse_mul/torch_kernel_cuda.cpp:10-38. Same module and function name; the tensors are handed
// to the C ABI of libonebitmul as raw device pointers.
//
// Differences from the reference binding, all on the side of doing what its Python caller means:
//   * both argument orders are taken -- the reference's C++ is onebit_mul(A, B, meta, C), its Python
//     calls onebit_mul(A, B, C, meta) (onebit_sparse_mul/__init__.py:14,18); meta is the int16 tensor;
//   * m, n, k come from meta and B (the reference reads m from A.size(0), which is k/2 for pack()'s
//     layout) and mismatching shapes raise (the reference raises when they MATCH, :17-18);
//   * the call runs on the current ATen stream of B's device; C may be float32 or float16.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "onebit_sparse_tensor.h"

namespace {

void onebit_mul_impl(const torch::Tensor& A, const torch::Tensor& B, const torch::Tensor& X, const torch::Tensor& Y,
                     const c10::optional<torch::Tensor>& scale) {
  const bool x_is_meta = X.scalar_type() == torch::kInt16;
  const torch::Tensor& meta = x_is_meta ? X : Y;
  const torch::Tensor& C = x_is_meta ? Y : X;
  TORCH_CHECK(meta.scalar_type() == torch::kInt16, "onebit_mul: meta must be int16");
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && meta.is_cuda() && C.is_cuda(), "onebit_mul: all tensors must be CUDA tensors");
  TORCH_CHECK(A.scalar_type() == torch::kUInt8, "onebit_mul: A must be uint8 (packed sign bits)");
  TORCH_CHECK(B.scalar_type() == torch::kHalf, "onebit_mul: B must be float16");
  TORCH_CHECK(C.scalar_type() == torch::kFloat || C.scalar_type() == torch::kHalf, "onebit_mul: C must be float32 or float16");
  TORCH_CHECK(A.is_contiguous() && B.is_contiguous() && meta.is_contiguous() && C.is_contiguous(), "onebit_mul: tensors must be contiguous");
  TORCH_CHECK(B.dim() == 2 && meta.dim() == 2 && C.dim() == 2, "onebit_mul: B, meta, C must be 2-dimensional");
  const int64_t m = meta.size(0), k = B.size(0), n = B.size(1);
  TORCH_CHECK(meta.size(1) * 16 == k, "onebit_mul: meta.size(1) * 16 != B.size(0)");
  TORCH_CHECK(A.numel() * 16 == m * k, "onebit_mul: A holds ", A.numel() * 8, " sign bits, expected ", m * k / 2);
  TORCH_CHECK(C.size(0) == m && C.size(1) == n, "onebit_mul: C must be (", m, ", ", n, ")");
  const void* scale_ptr = nullptr;
  torch::Tensor scale_t;
  if (scale.has_value() && scale->defined()) {
    scale_t = scale->to(B.device(), torch::kHalf).contiguous();
    TORCH_CHECK(scale_t.numel() == m, "onebit_mul: scale must have m elements");
    scale_ptr = scale_t.data_ptr();
  }
  c10::cuda::CUDAGuard guard(B.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t ws_bytes = (m % 128 == 0 && k % 128 == 0) ? (int64_t)onebit_workspace_bytes(m, k) : 0;
  torch::Tensor ws = torch::empty({std::max<int64_t>(ws_bytes, 256)}, torch::TensorOptions().dtype(torch::kUInt8).device(B.device()));
  const int rc = onebit_sparse_matmul_ex(A.data_ptr(), B.data_ptr(), C.data_ptr(), meta.data_ptr(), scale_ptr, m, n, k,
                                         C.scalar_type() == torch::kHalf ? ONEBIT_OUT_F16 : ONEBIT_OUT_F32, ONEBIT_META_PYTHON,
                                         ws_bytes ? ws.data_ptr() : nullptr, (size_t)ws_bytes, stream.stream());
  TORCH_CHECK(rc == ONEBIT_OK, "onebit_mul: ", onebit_last_error());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("onebit_mul", &onebit_mul_impl, "C = onebit 2:4 sparse A x fp16 B", pybind11::arg("A"), pybind11::arg("B"),
        pybind11::arg("meta_or_C"), pybind11::arg("C_or_meta"), pybind11::arg("scale") = c10::optional<torch::Tensor>());
}
