// Checker only: exposes the reference's own expert-grouped block-FP8 GEMM (compiled from the reference checkout where
// it lies, see oracle/Makefile target `ref_gpu_moe`) as torch.ops.sgl_gpu_ref.fp8_blockwise_scaled_grouped_mm, with
// the schema of sgl-kernel/csrc/common_extension.cc:253-257.  Used by tests/test_gpu_ref_kernel.py and the bench's
// comparator of the MoE section on one GPU; never by the product.
#include <torch/all.h>
#include <torch/library.h>
void fp8_blockwise_scaled_grouped_mm(torch::Tensor& output, torch::Tensor& a_ptrs, torch::Tensor& b_ptrs,
                                     torch::Tensor& out_ptrs, torch::Tensor& a_scales_ptrs, torch::Tensor& b_scales_ptrs,
                                     const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& scales_a,
                                     const torch::Tensor& scales_b, const torch::Tensor& stride_a,
                                     const torch::Tensor& stride_b, const torch::Tensor& stride_c,
                                     const torch::Tensor& layout_sfa, const torch::Tensor& layout_sfb,
                                     const torch::Tensor& problem_sizes, const torch::Tensor& expert_offsets,
                                     const torch::Tensor& workspace);
TORCH_LIBRARY_FRAGMENT(sgl_gpu_ref, m) {
  m.def(
      "fp8_blockwise_scaled_grouped_mm(Tensor output, Tensor a_ptrs, Tensor b_ptrs, Tensor out_ptrs, Tensor "
      "a_scales_ptrs, Tensor b_scales_ptrs, Tensor a, Tensor b, Tensor scales_a, Tensor scales_b, Tensor "
      "stride_a, Tensor stride_b, Tensor stride_c, Tensor layout_sfa, Tensor layout_sfb, Tensor problem_sizes, Tensor "
      "expert_offsets, Tensor workspace) -> ()");
  m.impl("fp8_blockwise_scaled_grouped_mm", torch::kCUDA, &fp8_blockwise_scaled_grouped_mm);
}
