// TEST/BENCH INFRASTRUCTURE ONLY -- never linked into or called by the product path.
//
// Registration shim for the reference's own CUDA kernels of the block-FP8 linear path, compiled
// where they lie by oracle/build_ref_cuda.py:
//   sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:345   fp8_blockwise_scaled_mm
//   sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:230  sgl_per_token_group_quant_fp8
//   sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu:587     fp8_blockwise_scaled_grouped_mm
//   sgl-kernel/csrc/moe/prepare_moe_input.cu                prepare_moe_input, shuffle_rows,
//                                                           apply_shuffle_mul_sum
// The operators are registered under the namespace `sgl_kernel_ref` (schemas as in
// sgl-kernel/csrc/common_extension.cc:111-119,192-207) so that they cannot collide with the
// product's `sgl_kernel::*` operators.  bench.py times them beside the product's kernels as the
// on-box comparator; nothing else uses them.
#include <ATen/ATen.h>
#include <torch/all.h>
#include <torch/library.h>

#include <optional>

torch::Tensor fp8_blockwise_scaled_mm(const torch::Tensor& mat_a, const torch::Tensor& mat_b,
                                      const torch::Tensor& scales_a, const torch::Tensor& scales_b,
                                      const torch::Dtype& out_dtype);
void sgl_per_token_group_quant_fp8(at::Tensor input, at::Tensor output_q, at::Tensor output_s, int64_t group_size,
                                   double eps, double fp8_min, double fp8_max, bool scale_ue8m0);
void fp8_blockwise_scaled_grouped_mm(torch::Tensor& output, torch::Tensor& a_ptrs, torch::Tensor& b_ptrs,
                                     torch::Tensor& out_ptrs, torch::Tensor& a_scales_ptrs,
                                     torch::Tensor& b_scales_ptrs, const torch::Tensor& a, const torch::Tensor& b,
                                     const torch::Tensor& scales_a, const torch::Tensor& scales_b,
                                     const torch::Tensor& stride_a, const torch::Tensor& stride_b,
                                     const torch::Tensor& stride_c, const torch::Tensor& layout_sfa,
                                     const torch::Tensor& layout_sfb, const torch::Tensor& problem_sizes,
                                     const torch::Tensor& expert_offsets, const torch::Tensor& workspace);
void prepare_moe_input(const torch::Tensor& topk_ids, torch::Tensor& expert_offsets,
                       const std::optional<torch::Tensor>& blockscale_offsets, torch::Tensor& problem_sizes1,
                       torch::Tensor& problem_sizes2, torch::Tensor& input_permutation,
                       torch::Tensor& output_permutation, const int64_t num_experts, const int64_t n,
                       const int64_t k);
void shuffle_rows(const torch::Tensor& input_tensor, const torch::Tensor& dst2src_map, torch::Tensor& output_tensor);
void apply_shuffle_mul_sum(const torch::Tensor& input, torch::Tensor& output, const torch::Tensor& permutation,
                           const std::optional<torch::Tensor>& factors);

TORCH_LIBRARY_FRAGMENT(sgl_kernel_ref, m) {
#ifdef REF_SHIM_GEMM
  m.def(
      "fp8_blockwise_scaled_mm(Tensor mat_a, Tensor mat_b, Tensor scales_a, Tensor scales_b, ScalarType out_dtype) -> "
      "Tensor");
  m.impl("fp8_blockwise_scaled_mm", torch::kCUDA, &fp8_blockwise_scaled_mm);
#endif
#ifdef REF_SHIM_QUANT
  m.def(
      "sgl_per_token_group_quant_fp8(Tensor input, Tensor output_q, Tensor output_s, int group_size, float eps, float "
      "fp8_min, float fp8_max, bool scale_ue8m0) -> ()");
  m.impl("sgl_per_token_group_quant_fp8", torch::kCUDA, &sgl_per_token_group_quant_fp8);
#endif
#ifdef REF_SHIM_MOE
  m.def(
      "fp8_blockwise_scaled_grouped_mm(Tensor output, Tensor a_ptrs, Tensor b_ptrs, Tensor out_ptrs, Tensor "
      "a_scales_ptrs, Tensor b_scales_ptrs, Tensor a, Tensor b, Tensor scales_a, Tensor scales_b, Tensor stride_a, "
      "Tensor stride_b, Tensor stride_c, Tensor layout_sfa, Tensor layout_sfb, Tensor problem_sizes, Tensor "
      "expert_offsets, Tensor workspace) -> ()");
  m.impl("fp8_blockwise_scaled_grouped_mm", torch::kCUDA, &fp8_blockwise_scaled_grouped_mm);
  m.def(
      "prepare_moe_input(Tensor topk_ids, Tensor expert_offsets, Tensor? blockscale_offsets, Tensor problem_sizes1, "
      "Tensor problem_sizes2, Tensor input_permutation, Tensor output_permutation, int num_experts, int n, int k) -> "
      "()");
  m.impl("prepare_moe_input", torch::kCUDA, &prepare_moe_input);
  m.def("shuffle_rows(Tensor input, Tensor dst2src_map, Tensor output) -> ()");
  m.impl("shuffle_rows", torch::kCUDA, &shuffle_rows);
  m.def("apply_shuffle_mul_sum(Tensor input, Tensor output, Tensor permutation, Tensor? factors) -> ()");
  m.impl("apply_shuffle_mul_sum", torch::kCUDA, &apply_shuffle_mul_sum);
#endif
}
