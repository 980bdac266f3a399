"""Counterpart of python/sglang/srt/layers/quantization/fp8_utils.py: the block-FP8 linear.

The reference picks among flashinfer / cutlass / aiter / deepgemm / triton at
start-up (`dispatch_w8a8_block_fp8_linear`, fp8_utils.py:151-161).  Here there
is one backend and nothing to select.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from .... import ops as _ops
from .fp8_kernel import per_token_group_quant_fp8


def b200_w8a8_block_fp8_linear(
    input: torch.Tensor,
    weight: torch.Tensor,
    block_size: List[int],
    weight_scale: torch.Tensor,
    input_scale: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Same contract as `triton_w8a8_block_fp8_linear` (fp8_utils.py:306-326), plus the
    pre-quantised input form (`input_scale` given) of the flashinfer/deepgemm variants (:164-194)."""
    input_2d = input.view(-1, input.shape[-1])
    output_shape = [*input.shape[:-1], weight.shape[0]]
    if input_scale is not None:
        q_input, x_scale = input_2d, input_scale.view(input_2d.shape[0], -1)
        out_dtype = torch.bfloat16
    else:
        q_input, x_scale = per_token_group_quant_fp8(input_2d, block_size[1], column_major_scales=False)
        out_dtype = input_2d.dtype
    output = _ops.w8a8_block_fp8_matmul(q_input, weight, x_scale, weight_scale, block_size, out_dtype, bias=bias)
    return output.view(*output_shape)


def dispatch_w8a8_block_fp8_linear() -> Callable:
    return b200_w8a8_block_fp8_linear
