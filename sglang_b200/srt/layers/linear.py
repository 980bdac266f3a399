"""Tensor-parallel linear layers that call `quant_method.apply` — the callers of the dense path.

After python/sglang/srt/layers/linear.py: `LinearBase` (:160-228), `ColumnParallelLinear` (:265-436),
`MergedColumnParallelLinear` (:439-800), `QKVParallelLinear` (:803-1195), `RowParallelLinear`
(:1198-1393).  Only what the block-FP8 path needs is kept: shapes per partition, sharding of a full
checkpoint tensor and of its 128x128 block scales (:737-746, :917-973: a shard of n output rows owns
n/128 scale rows, a shard of k input columns owns k/128 scale columns), and the all-reduce after a
row-parallel layer (:1384-1385).
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from ..distributed import (
    get_fused_row_parallel,
    get_tensor_model_parallel_rank,
    get_tensor_model_parallel_world_size,
    tensor_model_parallel_all_reduce,
)
from .quantization.fp8_kernel import per_token_group_quant_fp8


def divide(a: int, b: int) -> int:
    assert a % b == 0, f"{a} is not divisible by {b}"
    return a // b


class LinearBase(nn.Module):
    def __init__(self, input_size: int, output_size: int, params_dtype: torch.dtype = torch.bfloat16,
                 quant_config=None, prefix: str = ""):
        super().__init__()
        self.input_size = input_size
        self.output_size = output_size
        self.params_dtype = params_dtype
        self.quant_config = quant_config
        self.quant_method = quant_config.get_quant_method(self, prefix=prefix) if quant_config is not None else None
        if self.quant_method is None:
            raise NotImplementedError("this package implements the block-FP8 quantised linears only")
        self.tp_size = get_tensor_model_parallel_world_size()
        self.tp_rank = get_tensor_model_parallel_rank()


class ColumnParallelLinear(LinearBase):
    """Y = X W^T with W split along its output rows; the output stays sharded unless gather_output."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False, gather_output: bool = False,
                 params_dtype: torch.dtype = torch.bfloat16, quant_config=None,
                 output_sizes: Optional[List[int]] = None, prefix: str = "", device=None):
        super().__init__(input_size, output_size, params_dtype, quant_config, prefix)
        self.gather_output = gather_output
        self.output_sizes = output_sizes or [output_size]
        self.output_partition_sizes = [divide(s, self.tp_size) for s in self.output_sizes]
        self.output_size_per_partition = sum(self.output_partition_sizes)
        self.quant_method.create_weights(
            self, input_size, self.output_partition_sizes, input_size, output_size, params_dtype, device=device)
        self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, dtype=params_dtype, device=device),
                                 requires_grad=False) if bias else None

    def load_full_weight(self, weight: torch.Tensor, weight_scale_inv: torch.Tensor, block: int = 128) -> None:
        """Shards a full [N,K] e4m3 weight and its [N/128,K/128] scales; merged layers shard each logical
        part separately so that every rank holds its slice of every part (linear.py:737-746)."""
        w_parts, s_parts, off = [], [], 0
        for full, part in zip(self.output_sizes, self.output_partition_sizes):
            lo = off + self.tp_rank * part
            w_parts.append(weight[lo : lo + part])
            s_parts.append(weight_scale_inv[lo // block : (lo + part + block - 1) // block])
            off += full
        self.weight.data.copy_(torch.cat(w_parts, 0))
        self.weight_scale_inv.data.copy_(torch.cat(s_parts, 0))

    def forward(self, x):
        out = self.quant_method.apply(self, x, self.bias)
        if self.gather_output and self.tp_size > 1:
            from ..distributed import get_tp_group
            out = get_tp_group().all_gather(out, dim=-1)
        return out, None


class MergedColumnParallelLinear(ColumnParallelLinear):
    def __init__(self, input_size: int, output_sizes: List[int], **kw):
        super().__init__(input_size, sum(output_sizes), output_sizes=list(output_sizes), **kw)


class QKVParallelLinear(ColumnParallelLinear):
    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int, total_num_kv_heads: int, **kw):
        sizes = [total_num_heads * head_size, total_num_kv_heads * head_size, total_num_kv_heads * head_size]
        super().__init__(hidden_size, sum(sizes), output_sizes=sizes, **kw)


class RowParallelLinear(LinearBase):
    """Y = X W^T with W split along its input columns; partial outputs are summed by an all-reduce."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False, input_is_parallel: bool = True,
                 reduce_results: bool = True, params_dtype: torch.dtype = torch.bfloat16, quant_config=None,
                 prefix: str = "", device=None):
        super().__init__(input_size, output_size, params_dtype, quant_config, prefix)
        self.input_is_parallel = input_is_parallel
        self.reduce_results = reduce_results
        self.input_size_per_partition = divide(input_size, self.tp_size)
        self.quant_method.create_weights(
            self, self.input_size_per_partition, [output_size], input_size, output_size, params_dtype, device=device)
        self.bias = nn.Parameter(torch.zeros(output_size, dtype=params_dtype, device=device),
                                 requires_grad=False) if bias else None

    def load_full_weight(self, weight: torch.Tensor, weight_scale_inv: torch.Tensor, block: int = 128) -> None:
        k = self.input_size_per_partition
        lo = self.tp_rank * k
        self.weight.data.copy_(weight[:, lo : lo + k])
        self.weight_scale_inv.data.copy_(weight_scale_inv[:, lo // block : (lo + k + block - 1) // block])

    def forward(self, x):
        if not self.input_is_parallel and self.tp_size > 1:
            k = self.input_size_per_partition
            x = x[..., self.tp_rank * k : (self.tp_rank + 1) * k].contiguous()
        # bias is added by rank 0 only so that the all-reduce counts it once (linear.py:1376-1378)
        bias = self.bias if (self.tp_rank == 0 or self.tp_size == 1) else None
        fused = get_fused_row_parallel() if (self.reduce_results and self.tp_size > 1 and self.bias is None) else None
        if fused is not None and getattr(self.quant_method, "block_quant", False):
            # GEMM with the reduce-scatter in its epilogue, then one reduce-and-gather kernel over peer memory
            xq, xs = x if isinstance(x, tuple) else (None, None)
            lead = (xq if xq is not None else x).shape[:-1]
            rows = 1
            for d in lead:
                rows *= d
            if fused.supports(rows, self.output_size):
                if xq is None:
                    x2 = x.reshape(rows, x.shape[-1])
                    xq, xs = per_token_group_quant_fp8(x2, self.quant_method.quant_config.weight_block_size[1])
                    out_dtype = x.dtype
                else:
                    xq, xs, out_dtype = xq.reshape(rows, -1), xs.reshape(rows, -1), torch.bfloat16
                out = fused.linear(xq, xs, self.weight, self.weight_scale_inv, out_dtype)
                return out.view(*lead, self.output_size), None
        out = self.quant_method.apply(self, x, bias)
        if self.reduce_results and self.tp_size > 1:
            out = tensor_model_parallel_all_reduce(out)
        return out, None
