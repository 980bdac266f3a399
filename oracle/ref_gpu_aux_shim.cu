// Checker only: exposes the reference's own CUDA quantizer and its moe_align kernel (compiled from the reference
// checkout where they lie, see oracle/Makefile target `ref_gpu_aux`) as torch.ops.sgl_gpu_ref.*, with the schemas of
// sgl-kernel/csrc/common_extension.cc:138-141 and :218-222.  Used by tests/test_gpu_ref_kernel.py; never by the product.
#include <torch/all.h>
#include <torch/library.h>
void sgl_per_token_group_quant_8bit(torch::Tensor input, torch::Tensor output_q, torch::Tensor output_s,
                                    int64_t group_size, double eps, double min_8bit, double max_8bit, bool scale_ue8m0);
void moe_align_block_size(torch::Tensor topk_ids, int64_t num_experts, int64_t block_size,
                          torch::Tensor sorted_token_ids, torch::Tensor experts_ids, torch::Tensor num_tokens_post_pad,
                          torch::Tensor cumsum_buffer, bool pad_sorted_token_ids);
TORCH_LIBRARY_FRAGMENT(sgl_gpu_ref, m) {
  m.def(
      "sgl_per_token_group_quant_8bit(Tensor input, Tensor output_q, Tensor output_s, int group_size,"
      " float eps, float fp8_min, float fp8_max, bool scale_ue8m0) -> ()");
  m.impl("sgl_per_token_group_quant_8bit", torch::kCUDA, &sgl_per_token_group_quant_8bit);
  m.def(
      "moe_align_block_size(Tensor topk_ids, int num_experts, int block_size, Tensor! sorted_token_ids, Tensor! "
      "experts_ids, Tensor! num_tokens_post_pad, Tensor! cumsum_buffer, bool pad_sorted_token_ids) -> ()");
  m.impl("moe_align_block_size", torch::kCUDA, &moe_align_block_size);
}
