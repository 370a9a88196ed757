// TEST/BENCH INFRASTRUCTURE ONLY -- never linked into or called by the product path.
//
// Registration shim for the reference's own CPU block-FP8 matmul
// (sgl-kernel/csrc/cpu/gemm_fp8.cpp:468 `fp8_scaled_mm_cpu`, and the weight
// repacker sgl-kernel/csrc/cpu/gemm.cpp:401 `convert_weight_packed`).
// The two reference translation units are compiled where they lie by
// oracle/build_ref.py; this file only exposes them to Python under the
// namespace `sgl_kernel_ref` so they cannot collide with the product's
// `sgl_kernel::*` operators.
#include <torch/library.h>
#include <ATen/ATen.h>

#include <optional>
#include <vector>

at::Tensor convert_weight_packed(at::Tensor& weight);

at::Tensor fp8_scaled_mm_cpu(
    at::Tensor& mat1,
    at::Tensor& mat2,
    at::Tensor& scales2,
    std::vector<int64_t> block_size,
    const std::optional<at::Tensor>& bias,
    at::ScalarType out_dtype,
    bool is_vnni);

TORCH_LIBRARY_FRAGMENT(sgl_kernel_ref, m) {
  m.def("convert_weight_packed(Tensor weight) -> Tensor");
  m.impl("convert_weight_packed", c10::kCPU, &convert_weight_packed);
  m.def(
      "fp8_scaled_mm_cpu(Tensor mat1, Tensor mat2, Tensor scales2, int[] block_size, Tensor? bias, "
      "ScalarType out_dtype, bool is_vnni) -> Tensor");
  m.impl("fp8_scaled_mm_cpu", c10::kCPU, &fp8_scaled_mm_cpu);
}
