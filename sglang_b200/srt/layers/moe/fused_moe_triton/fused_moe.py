"""Counterpart of python/sglang/srt/layers/moe/fused_moe_triton/fused_moe.py for block-FP8 weights.

`fused_experts_impl` (:369-667) in the reference runs: moe_align -> quantise -> Triton grouped GEMM
(rows gathered in-kernel) -> silu_and_mul -> quantise -> Triton grouped GEMM (x top-k weight) ->
moe_sum_reduce.  Here the same steps run on the sm_100a kernels, with the two elementwise passes
between the GEMMs fused into one (silu_and_mul + re-quantisation) and the intermediate kept in
expert-sorted order so that both GEMMs read plain TMA tiles:

    quantise x            [T,H] bf16 -> e4m3 + 1x128 scales
    moe_align (block 128) topk_ids -> sorted_token_ids, expert_ids, num_tokens_post_pad
    gather rows           -> A1 [P,H] e4m3 (padding rows zero)
    grouped GEMM #1       -> ic1 [P,2I] bf16
    silu_and_mul+quantise -> A2 [P,I] e4m3 + scales
    grouped GEMM #2       -> ic3 [T*topk,H] bf16, scattered to token-major order, x top-k weight
    moe_sum_reduce        -> out [T,H]
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..... import ops as _ops

CHUNK_SIZE = 64 * 1024  # tokens per pass, as in the reference (:420)


def _max_padded_rows(numel: int, num_experts: int, block: int) -> int:
    # every non-empty bucket (at most min(numel, E+1) of them) adds at most block-1 padding rows
    rows = numel + min(numel, num_experts + 1) * (block - 1)
    return (rows + block - 1) // block * block


def fused_experts_impl(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    inplace: bool = False,
    activation: str = "silu",
    is_gated: bool = True,
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = True,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[List[int]] = None,
    no_combine: bool = False,
    routed_scaling_factor: Optional[float] = None,
    a1_scale: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
    has_filtered_ids: bool = False,
):
    """`a1_scale` given: `hidden_states` already holds e4m3 codes with these 1x128 scales (rows that
    arrived quantised from other ranks); the output dtype is then `out_dtype`.  `has_filtered_ids`: `topk_ids` may
    hold -1 (experts of other ranks, expert parallelism); their rows are then kept out of every kernel instead of
    being carried along and written as zeros."""
    if not use_fp8_w8a8 or block_shape is None or list(block_shape) != [128, 128]:
        raise NotImplementedError("only use_fp8_w8a8 with block_shape [128, 128] is on this path")
    if activation != "silu" or not is_gated:
        raise NotImplementedError("only the gated silu activation is on this path")
    assert hidden_states.shape[1] == w1.shape[2], "Hidden size mismatch"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.is_contiguous() and w2.is_contiguous(), "Expert weights must be contiguous"
    prequant = a1_scale is not None
    if prequant:
        assert hidden_states.dtype == torch.float8_e4m3fn and not inplace and not apply_router_weight_on_input
        act_dtype = out_dtype or torch.bfloat16
    else:
        assert hidden_states.dtype in (torch.float16, torch.bfloat16)
        act_dtype = hidden_states.dtype
    num_tokens, H = hidden_states.shape
    E, N, _ = w1.shape
    topk = topk_ids.shape[1]
    if routed_scaling_factor is None:
        routed_scaling_factor = 1.0
    if topk_ids.dtype != torch.int32:
        topk_ids = topk_ids.to(torch.int32)
    if topk_weights.dtype != torch.float32:
        topk_weights = topk_weights.float()

    if no_combine:
        assert not inplace
        out = torch.empty((num_tokens, topk, w2.shape[1]), device=hidden_states.device, dtype=act_dtype)
    elif inplace:
        out = hidden_states
    else:
        out = torch.empty((num_tokens, w2.shape[1]), device=hidden_states.device, dtype=act_dtype)

    for begin in range(0, num_tokens, CHUNK_SIZE):
        end = min(begin + CHUNK_SIZE, num_tokens)
        x = hidden_states[begin:end]
        ids = topk_ids[begin:end].contiguous()
        wts = topk_weights[begin:end].contiguous()
        t = end - begin
        numel = t * topk
        if apply_router_weight_on_input:
            assert topk == 1, "apply_router_weight_on_input is only implemented for topk=1"
            x = x * wts.to(x.dtype)
        if prequant:
            xq, xs = x, a1_scale[begin:end]
        else:
            xq, xs = _ops.per_token_group_quant_fp8(x, 128)
        direct = no_combine or (topk == 1 and routed_scaling_factor == 1.0)
        drop = has_filtered_ids and not direct  # (the direct forms need the zero rows of filtered slots in `out`)
        if drop:
            # rows of experts that live on other ranks (id -1) are dropped from the sorted order: they would only be
            # gathered, zero-filled and read back by every kernel below
            sorted_ids, expert_ids, post = _ops.moe_align_block_size_local(ids, _ops.ALIGN_BLOCK, E)
        else:
            sorted_ids, expert_ids, post = _ops.moe_align_block_size(ids, _ops.ALIGN_BLOCK, E)
        max_rows = _max_padded_rows(numel, E, _ops.ALIGN_BLOCK)
        a1, a1s = _ops.gather_rows_fp8(xq, xs, sorted_ids, post, numel, topk, max_rows)
        ic1 = _ops.grouped_block_fp8_matmul(a1, a1s, w1, w1_scale, sorted_ids, expert_ids, post, numel=numel,
                                            scatter=False, output_dtype=act_dtype)
        a2, a2s = _ops.silu_and_mul_quant_fp8(ic1, 128, num_rows=post)
        ic3 = out[begin:end].view(numel, -1) if direct else None
        ic3 = _ops.grouped_block_fp8_matmul(a2, a2s, w2, w2_scale, sorted_ids, expert_ids, post, numel=numel,
                                            scatter=True,
                                            row_weights=None if apply_router_weight_on_input else wts,
                                            out=ic3, output_dtype=act_dtype)
        if not direct:
            if drop:
                _ops.moe_sum_reduce_masked_out(ic3.view(t, topk, -1), ids, out[begin:end], routed_scaling_factor)
            else:
                _ops.moe_sum_reduce_out(ic3.view(t, topk, -1), out[begin:end], routed_scaling_factor)
    return out


def fused_experts(hidden_states, w13_weight, w2_weight, topk_output, moe_runner_config, *, w13_scale, w2_scale,
                  block_shape, has_filtered_ids: bool = False):
    """`fused_experts` (:261-319) with the quantisation info spelled out."""
    topk_weights, topk_ids = topk_output[0], topk_output[1]
    return fused_experts_impl(
        hidden_states, w13_weight, w2_weight, topk_weights, topk_ids,
        inplace=moe_runner_config.inplace and not moe_runner_config.no_combine,
        activation=moe_runner_config.activation, is_gated=moe_runner_config.is_gated,
        apply_router_weight_on_input=moe_runner_config.apply_router_weight_on_input,
        use_fp8_w8a8=True, w1_scale=w13_scale, w2_scale=w2_scale, block_shape=block_shape,
        no_combine=moe_runner_config.no_combine, routed_scaling_factor=moe_runner_config.routed_scaling_factor,
        has_filtered_ids=has_filtered_ids,
    )
