"""The masked expert layout of the expert-parallel MoE path.

After python/sglang/srt/layers/moe/ep_moe/kernels.py:287-420 (`_silu_and_mul_post_quant_kernel`,
`silu_and_mul_masked_post_quant_fwd`): the output of the first grouped GEMM arrives as
[experts, padded tokens, 2 x intermediate] with `masked_m[e]` valid rows per expert; gate and up halves are combined
(silu in float32, rounded to the tensor type, times up in that type) and re-quantised per 128 columns for the second
grouped GEMM.  One kernel of this library does that (`sglb200_silu_and_mul_masked_quant_fp8`); the scales are
float32 (`scale_ue8m0=True` belongs to the DeepGEMM path and raises).
"""
from __future__ import annotations

import torch

from ..... import ops as _ops


def silu_and_mul_masked_post_quant_fwd(input: torch.Tensor, output: torch.Tensor, output_scale: torch.Tensor,
                                       quant_group_size: int, masked_m: torch.Tensor, scale_ue8m0: bool = False) -> None:
    """input [expert_num, token_num_padded, hidden_dim]; output [expert_num, token_num_padded, hidden_dim // 2] fp8;
    output_scale [expert_num, token_num_padded, hidden_dim // 2 // quant_group_size] float32; masked_m [expert_num].
    Rows at or beyond masked_m[e] are left as they are."""
    if scale_ue8m0:
        raise NotImplementedError("UE8M0 scales belong to the DeepGEMM path, which this library does not serve")
    assert input.is_contiguous()
    assert output.dtype == torch.float8_e4m3fn
    assert output.is_contiguous()
    assert len(input.shape) == 3
    assert input.shape[0] == masked_m.shape[0]
    assert input.shape[-1] % 2 == 0
    assert (input.shape[-1] // 2) % quant_group_size == 0
    _ops.silu_and_mul_masked_quant_fp8_out(input, output, output_scale, masked_m.to(torch.int32), quant_group_size)
