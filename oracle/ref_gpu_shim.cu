// Checker only: exposes the reference's own CUDA block-FP8 GEMM (compiled from the reference checkout where it
// lies, see oracle/Makefile target `ref_gpu`) as torch.ops.sgl_gpu_ref.fp8_blockwise_scaled_mm, with the schema of
// sgl-kernel/csrc/common_extension.cc:133-136.  Used by tests/test_gpu_ref_kernel.py and the bench's comparator
// section; never by the product.
#include <torch/all.h>
#include <torch/library.h>
torch::Tensor fp8_blockwise_scaled_mm(const torch::Tensor& mat_a, const torch::Tensor& mat_b, const torch::Tensor& scales_a,
                                      const torch::Tensor& scales_b, const torch::Dtype& out_dtype);
TORCH_LIBRARY_FRAGMENT(sgl_gpu_ref, m) {
  m.def("fp8_blockwise_scaled_mm(Tensor mat_a, Tensor mat_b, Tensor scales_a, Tensor scales_b, ScalarType out_dtype) -> Tensor");
  m.impl("fp8_blockwise_scaled_mm", torch::kCUDA, &fp8_blockwise_scaled_mm);
}
