"""Drop-in for the `sgl_kernel` Python package, restricted to the block-FP8 path.

Importing this module registers the ops under `torch.ops.sgl_kernel.*` with the
reference's schemas (sgl-kernel/csrc/common_extension.cc:78-79,133-141,218-222,
234-235,263-264) so that callers written against the reference
(`torch.ops.sgl_kernel.moe_align_block_size.default(...)`) run unchanged, and
exposes the reference's Python-level function names.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops as _ops

_SCHEMAS = {
    "fp8_blockwise_scaled_mm": "(Tensor mat_a, Tensor mat_b, Tensor scales_a, Tensor scales_b, ScalarType out_dtype) -> Tensor",
    "sgl_per_token_group_quant_8bit": "(Tensor input, Tensor(a!) output_q, Tensor(b!) output_s, int group_size, float eps, float fp8_min, float fp8_max, bool scale_ue8m0) -> ()",
    "sgl_per_token_group_quant_8bit_v2": "(Tensor input, Tensor(a!) output_q, Tensor(b!) output_s, int group_size, float eps, float fp8_min, float fp8_max, bool scale_ue8m0, bool fuse_silu_and_mul, Tensor? masked_m) -> ()",
    "moe_align_block_size": "(Tensor topk_ids, int num_experts, int block_size, Tensor(a!) sorted_token_ids, Tensor(b!) experts_ids, Tensor(c!) num_tokens_post_pad, Tensor(d!) cumsum_buffer, bool pad_sorted_token_ids) -> ()",
    "silu_and_mul": "(Tensor(a!) out, Tensor input) -> ()",
    "moe_sum_reduce": "(Tensor input, Tensor(a!) output, float routed_scaling_factor) -> ()",
    "shuffle_rows": "(Tensor input, Tensor dst2src_map, Tensor(a!) output) -> ()",
    "apply_shuffle_mul_sum": "(Tensor input, Tensor(a!) output, Tensor permutation, Tensor? factors) -> ()",
    "prepare_moe_input": "(Tensor topk_ids, Tensor(a!) expert_offsets, Tensor(b!)? blockscale_offsets, Tensor(c!) problem_sizes1, Tensor(d!) problem_sizes2, Tensor(e!) input_permutation, Tensor(f!) output_permutation, int num_experts, int n, int k) -> ()",
    "fp8_blockwise_scaled_grouped_mm": "(Tensor(a!) output, Tensor a_ptrs, Tensor b_ptrs, Tensor out_ptrs, Tensor a_scales_ptrs, Tensor b_scales_ptrs, Tensor a, Tensor b, Tensor scales_a, Tensor scales_b, Tensor stride_a, Tensor stride_b, Tensor stride_c, Tensor layout_sfa, Tensor layout_sfb, Tensor problem_sizes, Tensor expert_offsets, Tensor workspace) -> ()",
    "topk_softmax": "(Tensor(a!) topk_weights, Tensor(b!) topk_indices, Tensor gating_output, bool renormalize, float moe_softcapping, Tensor? correction_bias) -> ()",
    "topk_sigmoid": "(Tensor(a!) topk_weights, Tensor(b!) topk_indices, Tensor gating_output, bool renormalize, Tensor? correction_bias) -> ()",
    "moe_fused_gate": "(Tensor input, Tensor bias, int num_expert_group, int topk_group, int topk, int num_fused_shared_experts, float routed_scaling_factor, bool apply_routed_scaling_factor_on_output) -> Tensor[]",
}


def _op_fp8_blockwise_scaled_mm(mat_a, mat_b, scales_a, scales_b, out_dtype):
    # Reference layout (fp8_blockwise_gemm_kernel.cu:374-406): mat_a [M,K] row-major, mat_b [K,N] column-major
    # (= weight.T), scales_a [M,K/128] M-major, scales_b [K/128,N/128] (= weight_scale.T).
    if mat_b.stride(0) != 1:
        raise RuntimeError("mat_b must be a column-major tensor")
    if mat_a.stride(1) != 1:
        raise RuntimeError("mat_a must be a row-major tensor")
    weight = mat_b.t()  # [N,K] contiguous view
    return _ops.w8a8_block_fp8_matmul(mat_a, weight, scales_a, scales_b.t(), [128, 128], out_dtype)


def _op_quant(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0):
    if scale_ue8m0:
        raise NotImplementedError("UE8M0 scales are not part of this path (float32 128-block scales only)")
    _ops.per_token_group_quant_fp8_out(input, output_q, output_s, group_size, eps, fp8_min, fp8_max)


def _op_quant_v2(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, fuse_silu_and_mul, masked_m):
    if scale_ue8m0 or masked_m is not None:
        raise NotImplementedError("UE8M0 scales / masked layout are not part of this path")
    if not fuse_silu_and_mul:
        return _op_quant(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, False)
    if not output_s.is_contiguous():
        raise NotImplementedError("fused silu_and_mul quantisation writes row-major scales")
    q, s = _ops.silu_and_mul_quant_fp8(input, group_size, eps)
    output_q.copy_(q)
    output_s.copy_(s)


def _op_moe_align(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad, cumsum_buffer, pad_sorted_token_ids):
    _ops.moe_align_block_size_out(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids,
                                  num_tokens_post_pad, cumsum_buffer, pad_sorted_token_ids)


def _op_silu_and_mul(out, input):
    _ops.silu_and_mul_out(out, input)


def _op_moe_sum_reduce(input, output, routed_scaling_factor):
    _ops.moe_sum_reduce_out(input, output, routed_scaling_factor)


def _op_shuffle_rows(input, dst2src_map, output):
    # prepare_moe_input.cu:170-197: output[i, :] = input[dst2src_map[i], :]; plain row gather.
    src = input.view(torch.uint8) if input.dtype.itemsize == 1 else input
    dst = output.view(torch.uint8) if output.dtype.itemsize == 1 else output
    torch.index_select(src, 0, dst2src_map.long(), out=dst)


def _op_apply_shuffle_mul_sum(input, output, permutation, factors):
    _ops.shuffle_mul_sum_out(input, output, permutation.reshape(-1), None if factors is None else factors.reshape(-1))


def _op_prepare_moe_input(topk_ids, expert_offsets, blockscale_offsets, problem_sizes1, problem_sizes2,
                          input_permutation, output_permutation, num_experts, n, k):
    # prepare_moe_input.cu:10-168: rows per expert, their prefix sums, and the two permutations between the
    # token-major and the expert-major order.  The reference fills the permutations with atomics (any order inside
    # an expert); here the order is the stable one of this library's sort (block size 1 = no padding).
    if topk_ids.dtype != torch.int32:
        raise RuntimeError("prepare_moe_input: topk_ids must be int32")
    numel, topk = topk_ids.numel(), topk_ids.shape[1]
    order, _, _ = _ops.moe_align_block_size(topk_ids, 1, num_experts)
    order = order[:numel]
    # rows per expert without a data-dependent shape (nothing synchronises, negative ids = filtered slots are
    # counted in a bucket of their own and dropped)
    counts = torch.zeros(num_experts + 1, dtype=torch.int32, device=topk_ids.device)
    flat = topk_ids.reshape(-1)
    bucket = torch.where((flat >= 0) & (flat < num_experts), flat + 1, torch.zeros_like(flat)).long()
    counts.scatter_add_(0, bucket, torch.ones_like(flat))
    counts = counts[1:]
    expert_offsets[0] = 0
    expert_offsets[1 : num_experts + 1] = torch.cumsum(counts, 0)
    if blockscale_offsets is not None:
        blockscale_offsets[0] = 0
        blockscale_offsets[1 : num_experts + 1] = torch.cumsum((counts + 127) // 128 * 128, 0)
    problem_sizes1[:, 0], problem_sizes1[:, 1], problem_sizes1[:, 2] = counts, 2 * n, k
    problem_sizes2[:, 0], problem_sizes2[:, 1], problem_sizes2[:, 2] = counts, k, n
    input_permutation.copy_(order // topk)
    output_permutation[order.long()] = torch.arange(numel, dtype=torch.int32, device=topk_ids.device)


def _op_fp8_blockwise_scaled_grouped_mm(output, a_ptrs, b_ptrs, out_ptrs, a_scales_ptrs, b_scales_ptrs, a, b, scales_a,
                                        scales_b, stride_a, stride_b, stride_c, layout_sfa, layout_sfb, problem_sizes,
                                        expert_offsets, workspace):
    # fp8_blockwise_moe_kernel.cu:650-810: per expert e, output[off_e : off_e + M_e] = blockscaled(a[off_e : ...], b[e]).
    # The pointer / stride / layout / workspace tensors are scratch of the reference's CUTLASS launch and are not
    # needed here.  The rows of every expert are padded to this library's 128-row blocks (stable sort of the rows'
    # expert numbers), gathered, multiplied, and written back to their unpadded places by the scatter epilogue.
    R, K = a.shape
    E = b.shape[0]
    w = b.transpose(1, 2)  # the reference passes [E, K, N] views of [E, N, K] weights
    if not w.is_contiguous():
        raise RuntimeError("fp8_blockwise_scaled_grouped_mm: b must be the transposed view of a contiguous [E, N, K] tensor")
    N = w.shape[1]
    nb, kb = (N + 127) // 128, (K + 127) // 128
    if scales_b.transpose(1, 2).is_contiguous() and tuple(scales_b.shape[1:]) == (kb, nb):
        ws = scales_b.transpose(1, 2)  # as fp8.py passes them: the transposed view of [E, N/128, K/128]
    elif scales_b.is_contiguous() and tuple(scales_b.shape[1:]) == (nb, kb):
        ws = scales_b
    else:
        raise RuntimeError("fp8_blockwise_scaled_grouped_mm: scales_b must be [E, N/128, K/128] or its transposed view")
    rows_per_expert = problem_sizes[:, 0].to(torch.int64)
    row_expert = torch.repeat_interleave(torch.arange(E, device=a.device, dtype=torch.int32), rows_per_expert,
                                         output_size=R)
    sorted_ids, expert_ids, post = _ops.moe_align_block_size(row_expert.view(R, 1), 128, E)
    aq, a_s = _ops.gather_rows_fp8(a, scales_a.contiguous(), sorted_ids, post, R, 1)
    _ops.grouped_block_fp8_matmul(aq, a_s, w, ws, sorted_ids, expert_ids, post, numel=R, scatter=True, out=output)


def _op_topk_softmax(topk_weights, topk_indices, gating_output, renormalize, moe_softcapping, correction_bias):
    _ops.topk_softmax_out(topk_weights, topk_indices, gating_output, renormalize, moe_softcapping, correction_bias)


def _op_topk_sigmoid(topk_weights, topk_indices, gating_output, renormalize, correction_bias):
    _ops.topk_sigmoid_out(topk_weights, topk_indices, gating_output, renormalize, correction_bias)


def _op_moe_fused_gate(input, bias, num_expert_group, topk_group, topk, num_fused_shared_experts,
                       routed_scaling_factor, apply_routed_scaling_factor_on_output):
    w, ids = _ops.moe_fused_gate(input, bias, num_expert_group, topk_group, topk, num_fused_shared_experts,
                                 routed_scaling_factor, apply_routed_scaling_factor_on_output)
    return [w, ids]


_IMPLS = {
    "fp8_blockwise_scaled_mm": _op_fp8_blockwise_scaled_mm,
    "sgl_per_token_group_quant_8bit": _op_quant,
    "sgl_per_token_group_quant_8bit_v2": _op_quant_v2,
    "moe_align_block_size": _op_moe_align,
    "silu_and_mul": _op_silu_and_mul,
    "moe_sum_reduce": _op_moe_sum_reduce,
    "shuffle_rows": _op_shuffle_rows,
    "apply_shuffle_mul_sum": _op_apply_shuffle_mul_sum,
    "prepare_moe_input": _op_prepare_moe_input,
    "fp8_blockwise_scaled_grouped_mm": _op_fp8_blockwise_scaled_grouped_mm,
    "topk_softmax": _op_topk_softmax,
    "topk_sigmoid": _op_topk_sigmoid,
    "moe_fused_gate": _op_moe_fused_gate,
}

def _fake_none(*args, **kwargs):
    return None


def _fake_fp8_blockwise_scaled_mm(mat_a, mat_b, scales_a, scales_b, out_dtype):
    return mat_a.new_empty((mat_a.shape[0], mat_b.shape[1]), dtype=out_dtype)


def _fake_moe_fused_gate(input, bias, num_expert_group, topk_group, topk, num_fused_shared_experts,
                         routed_scaling_factor, apply_routed_scaling_factor_on_output):
    return [input.new_empty((input.shape[0], topk), dtype=torch.float32),
            input.new_empty((input.shape[0], topk), dtype=torch.int32)]


_FAKES = {"fp8_blockwise_scaled_mm": _fake_fp8_blockwise_scaled_mm, "moe_fused_gate": _fake_moe_fused_gate}

_LIBRARY = None


def _register():
    global _LIBRARY
    if _LIBRARY is not None:
        return
    lib = torch.library.Library("sgl_kernel", "FRAGMENT")
    for name, schema in _SCHEMAS.items():
        lib.define(name + schema)
        lib.impl(name, _IMPLS[name], "CUDA")
        # shape-only implementations for tracing (torch.compile, FakeTensor, meta tensors), as the reference
        # registers for its ops (fp8_kernel.py:48-50, 1840-1859; fp8_utils.py:58-63)
        torch.library.register_fake(f"sgl_kernel::{name}", _FAKES.get(name, _fake_none), lib=lib)
    _LIBRARY = lib


_register()

# ---- Python-level names (sgl_kernel/gemm.py:25,100-140; moe.py:6,83; elementwise.py:172) ----


def fp8_blockwise_scaled_mm(mat_a, mat_b, scales_a, scales_b, out_dtype):
    return torch.ops.sgl_kernel.fp8_blockwise_scaled_mm.default(mat_a, mat_b, scales_a, scales_b, out_dtype)


def sgl_per_token_group_quant_8bit(input, output_q, output_s, group_size, eps, fp8_min, fp8_max,
                                   scale_ue8m0: bool = False, fuse_silu_and_mul: bool = False,
                                   masked_m: Optional[torch.Tensor] = None, enable_v2: Optional[bool] = None) -> None:
    if enable_v2 or fuse_silu_and_mul or masked_m is not None:
        return torch.ops.sgl_kernel.sgl_per_token_group_quant_8bit_v2.default(
            input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, fuse_silu_and_mul, masked_m)
    torch.ops.sgl_kernel.sgl_per_token_group_quant_8bit.default(
        input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0)


sgl_per_token_group_quant_fp8 = sgl_per_token_group_quant_8bit


def moe_align_block_size(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad,
                         cumsum_buffer, pad_sorted_token_ids=False):
    torch.ops.sgl_kernel.moe_align_block_size.default(
        topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad, cumsum_buffer,
        pad_sorted_token_ids)


def prepare_moe_input(topk_ids, expert_offsets, problem_sizes1, problem_sizes2, input_permutation, output_permutation,
                      num_experts, n, k, blockscale_offsets=None):
    torch.ops.sgl_kernel.prepare_moe_input.default(topk_ids, expert_offsets, blockscale_offsets, problem_sizes1,
                                                   problem_sizes2, input_permutation, output_permutation, num_experts,
                                                   n, k)


def apply_shuffle_mul_sum(input, output, permutation, factors=None):
    torch.ops.sgl_kernel.apply_shuffle_mul_sum.default(input, output, permutation, factors)


def fp8_blockwise_scaled_grouped_mm(output, a_ptrs, b_ptrs, out_ptrs, a_scales_ptrs, b_scales_ptrs, a, b, scales_a, scales_b,
                                    stride_a, stride_b, stride_c, layout_sfa, layout_sfb, problem_sizes, expert_offsets,
                                    workspace):
    torch.ops.sgl_kernel.fp8_blockwise_scaled_grouped_mm.default(
        output, a_ptrs, b_ptrs, out_ptrs, a_scales_ptrs, b_scales_ptrs, a, b, scales_a, scales_b, stride_a, stride_b,
        stride_c, layout_sfa, layout_sfb, problem_sizes, expert_offsets, workspace)


def topk_softmax(topk_weights, topk_ids, gating_output, renormalize=False, moe_softcapping=0.0, correction_bias=None) -> None:
    torch.ops.sgl_kernel.topk_softmax.default(topk_weights, topk_ids, gating_output, renormalize, moe_softcapping,
                                              correction_bias)


def topk_sigmoid(topk_weights, topk_ids, gating_output, renormalize=False, correction_bias=None) -> None:
    torch.ops.sgl_kernel.topk_sigmoid.default(topk_weights, topk_ids, gating_output, renormalize, correction_bias)


def moe_fused_gate(input_tensor, bias, num_expert_group, topk_group, topk, num_fused_shared_experts=0,
                   routed_scaling_factor=0, apply_routed_scaling_factor_on_output=False):
    return torch.ops.sgl_kernel.moe_fused_gate.default(input_tensor, bias, num_expert_group, topk_group, topk,
                                                       num_fused_shared_experts, routed_scaling_factor,
                                                       apply_routed_scaling_factor_on_output)


def moe_sum_reduce(input_tensor, output_tensor, routed_scaling_factor=0):
    torch.ops.sgl_kernel.moe_sum_reduce.default(input_tensor, output_tensor, routed_scaling_factor)


def silu_and_mul(input: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    if input.shape[-1] * input.dtype.itemsize % 16 != 0:
        raise ValueError("The pointers must be multiple of 16 bytes.")
    if out is None:
        out = torch.empty(input.shape[:-1] + (input.shape[-1] // 2,), device=input.device, dtype=input.dtype)
    else:
        assert input.shape[:-1] == out.shape[:-1] and input.shape[-1] == 2 * out.shape[-1]
    torch.ops.sgl_kernel.silu_and_mul.default(out, input)
    return out


def shuffle_rows(input_tensor, dst2src_map, output_tensor_shape):
    output = torch.empty(output_tensor_shape, device=input_tensor.device, dtype=input_tensor.dtype)
    torch.ops.sgl_kernel.shuffle_rows.default(input_tensor, dst2src_map, output)
    return output
