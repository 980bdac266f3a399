"""Counterpart of python/sglang/srt/layers/quantization/fp8_kernel.py for the block-FP8 path.

Same function names and argument meaning; one implementation (the sm_100a CUDA
library) instead of the Triton kernels (:125-216, :695-777), the sgl_kernel v1/v2
quantizers and the DeepGEMM dispatch (:1153-1168).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .... import ops as _ops

fp8_dtype = torch.float8_e4m3fn
fp8_max = torch.finfo(fp8_dtype).max
fp8_min = -fp8_max


def create_per_token_group_quant_fp8_output_scale(
    x_shape, device, group_size, column_major_scales: bool, scale_tma_aligned: bool, scale_ue8m0: bool
):
    """Scale tensor layouts of fp8_kernel.py:437-478 (float32 only: UE8M0 packing is not on this path)."""
    if scale_ue8m0:
        raise NotImplementedError("UE8M0 scales are not part of the float32 128-block path")
    if column_major_scales:
        if scale_tma_aligned:
            aligned_size = (x_shape[-2] + 3) // 4 * 4
            return torch.empty(
                x_shape[:-2] + (x_shape[-1] // group_size, aligned_size), device=device, dtype=torch.float32
            ).transpose(-1, -2)[: x_shape[-2], :]
        return torch.empty(
            (x_shape[-1] // group_size,) + x_shape[:-1], device=device, dtype=torch.float32
        ).permute(-1, -2)
    return torch.empty(x_shape[:-1] + (x_shape[-1] // group_size,), device=device, dtype=torch.float32)


def per_token_group_quant_fp8(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    dtype: torch.dtype = fp8_dtype,
    column_major_scales: bool = False,
    scale_tma_aligned: bool = False,
    scale_ue8m0: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp8_kernel.py:219-327 (`_per_token_group_quant_8bit_raw`)."""
    assert x.shape[-1] % group_size == 0, "the last dimension of `x` cannot be divisible by `group_size`"
    assert x.is_contiguous(), "`x` is not contiguous"
    if dtype != fp8_dtype:
        raise NotImplementedError("only float8_e4m3fn output is on this path")
    x_q = torch.empty_like(x, device=x.device, dtype=dtype)
    x_s = create_per_token_group_quant_fp8_output_scale(
        x.shape, x.device, group_size, column_major_scales, scale_tma_aligned, scale_ue8m0
    )
    if x.numel() > 0:
        x2 = x.view(-1, x.shape[-1])
        s2 = x_s if x_s.dim() == 2 else x_s.reshape(-1, x_s.shape[-1])
        _ops.per_token_group_quant_fp8_out(x2, x_q.view(-1, x.shape[-1]), s2, group_size, eps, fp8_min, fp8_max)
    return x_q, x_s


def sglang_per_token_group_quant_fp8(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    column_major_scales: bool = False,
    scale_tma_aligned: bool = False,
    scale_ue8m0: bool = False,
    fuse_silu_and_mul: bool = False,
    masked_m: Optional[torch.Tensor] = None,
    enable_v2: Optional[bool] = None,
):
    """fp8_kernel.py:481-531."""
    assert x.shape[-1] % group_size == 0, "the last dimension of `x` cannot be divisible by `group_size`"
    assert x.is_contiguous(), "`x` is not contiguous"
    if masked_m is not None:
        # fp8_kernel.py:329-403: the reference serves this combination only with UE8M0 scales in DeepGEMM's packed
        # layout (it asserts column_major_scales, scale_tma_aligned and scale_ue8m0), which this library does not
        # produce.  The masked layout with float32 scales is `silu_and_mul_masked_post_quant_fwd`
        # (srt/layers/moe/ep_moe/kernels.py), as in the reference.
        raise NotImplementedError("masked_m goes with UE8M0 scales in the reference's per_token_group_quant_8bit; "
                                  "for float32 scales call ep_moe.kernels.silu_and_mul_masked_post_quant_fwd")
    if fuse_silu_and_mul:
        if column_major_scales or scale_ue8m0:
            raise NotImplementedError("fused silu_and_mul quantisation writes row-major float32 scales")
        return _ops.silu_and_mul_quant_fp8(x, group_size, eps)
    return per_token_group_quant_fp8(
        x, group_size, eps, column_major_scales=column_major_scales, scale_tma_aligned=scale_tma_aligned,
        scale_ue8m0=scale_ue8m0,
    )


def w8a8_block_fp8_matmul(
    A: torch.Tensor,
    B: torch.Tensor,
    As: torch.Tensor,
    Bs: torch.Tensor,
    block_size: List[int],
    output_dtype: torch.dtype = torch.float16,
) -> torch.Tensor:
    """fp8_kernel.py:1153-1168: A [..., K] e4m3, B [N, K] e4m3, As [..., K/128], Bs [N/128, K/128]."""
    assert len(block_size) == 2
    assert A.shape[-1] == B.shape[-1]
    assert A.shape[:-1] == As.shape[:-1] and A.is_contiguous()
    assert B.ndim == 2 and B.is_contiguous() and Bs.ndim == 2
    return _ops.w8a8_block_fp8_matmul(A, B, As, Bs, block_size, output_dtype)


w8a8_block_fp8_matmul_triton = w8a8_block_fp8_matmul  # name kept for callers of the Triton variant (:1072)
