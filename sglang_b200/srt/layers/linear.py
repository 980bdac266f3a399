"""Tensor-parallel linear layers that call `quant_method.apply` — the callers of the dense path.

After python/sglang/srt/layers/linear.py: `LinearBase` (:160-228), `ColumnParallelLinear` (:265-436),
`MergedColumnParallelLinear` (:439-800), `QKVParallelLinear` (:803-1195), `RowParallelLinear`
(:1198-1393).  Only what the block-FP8 path needs is kept: shapes per partition, sharding of a full
checkpoint tensor and of its 128x128 block scales (:737-746, :917-973: a shard of n output rows owns
n/128 scale rows, a shard of k input columns owns k/128 scale columns), and the all-reduce after a
row-parallel layer (:1384-1385).

Checkpoint loading: every layer gives its `weight` and `weight_scale_inv` parameters a `weight_loader` attribute with
the calling convention of the reference's loaders (`param.weight_loader(param, loaded_weight[, shard_id])`,
:381-436, :575-763, :1035-1195, :1314-1352) so that a model's `load_weights` loop can drive them
(`srt/model_loader/weight_utils.py`).  `loaded_weight` is the FULL checkpoint tensor of one logical matrix; the
loader keeps this rank's rows or columns, and 1/128 of them (rounded up) for a block-scale parameter.
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


def _ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def _copy_checked(dst: torch.Tensor, src: torch.Tensor, what: str) -> None:
    if tuple(dst.shape) != tuple(src.shape):
        raise ValueError(f"{what}: checkpoint shard of shape {tuple(src.shape)} does not fit the parameter slice "
                         f"of shape {tuple(dst.shape)}")
    if dst.dtype == torch.float8_e4m3fn:  # copy codes as bytes (no float8 copy kernels are needed on any device)
        if src.dtype != torch.float8_e4m3fn:
            raise ValueError(f"{what}: the checkpoint holds {src.dtype}, the layer wants serialized float8_e4m3fn")
        dst.view(torch.uint8).copy_(src.view(torch.uint8))
    else:
        dst.copy_(src)


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
        self.prefix = prefix

    def _attach_loaders(self) -> None:
        for name in ("weight", "weight_scale_inv"):
            param = getattr(self, name)
            param.weight_loader = self.weight_loader
            param.is_block_scale = name == "weight_scale_inv"

    def _block(self, param) -> tuple:
        """(rows, columns) of the weight that one element of `param` stands for."""
        if getattr(param, "is_block_scale", False):
            bn, bk = self.quant_method.quant_config.weight_block_size
            return bn, bk
        return 1, 1


class ReplicatedLinear(LinearBase):
    """Y = X W^T with the whole W on every rank (linear.py:231-262); DeepSeek's fused_qkv_a_proj_with_mqa is one."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False, params_dtype: torch.dtype = torch.bfloat16,
                 quant_config=None, prefix: str = "", device=None):
        super().__init__(input_size, output_size, params_dtype, quant_config, prefix)
        # (partition sizes equal to the full sizes: none of create_weights' tensor-parallel divisibility rules
        # applies, so an output size like 2112 = 16.5 blocks is accepted, as by the reference's replicated layer)
        self.tp_size, self.tp_rank = 1, 0
        self.quant_method.create_weights(self, input_size, [output_size], input_size, output_size, params_dtype,
                                         device=device)
        self.bias = nn.Parameter(torch.zeros(output_size, dtype=params_dtype, device=device),
                                 requires_grad=False) if bias else None
        self._attach_loaders()

    def weight_loader(self, param, loaded_weight: torch.Tensor) -> None:
        _copy_checked(param.data, loaded_weight, self.prefix or "ReplicatedLinear")

    def forward(self, x):
        return self.quant_method.apply(self, x, self.bias), None


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
        self._attach_loaders()

    def _load_part(self, param, loaded_weight: torch.Tensor, part: int, src_block: Optional[int] = None) -> None:
        """Logical part `part` of a (merged) column-parallel parameter from the full tensor of that part:
        destination rows [sum of the earlier parts, + this part) of this rank's shard, source rows
        [src_block x this part, + this part); rows counted in 128-row blocks, rounded up, for a scale parameter
        (linear.py:737-746).  `src_block` defaults to this rank (a replicated KV head passes its own index)."""
        bn, _ = self._block(param)
        size = _ceil_div(self.output_partition_sizes[part], bn)
        dst_off = _ceil_div(sum(self.output_partition_sizes[:part]), bn)
        src_off = (self.tp_rank if src_block is None else src_block) * size
        if src_off + size > loaded_weight.shape[0]:
            raise ValueError(f"{self.prefix}: rows {src_off}..{src_off + size} of a checkpoint tensor with "
                             f"{loaded_weight.shape[0]} rows")
        _copy_checked(param.data.narrow(0, dst_off, size), loaded_weight.narrow(0, src_off, size), self.prefix)

    def weight_loader(self, param, loaded_weight: torch.Tensor, loaded_shard_id: Optional[int] = None) -> None:
        """`loaded_shard_id` None: the checkpoint tensor holds all logical parts one after the other (a plain
        column-parallel layer, or a merged one stored fused on disk: linear.py:651-707); an int: it holds that part."""
        if loaded_shard_id is not None:
            assert 0 <= loaded_shard_id < len(self.output_sizes)
            self._load_part(param, loaded_weight, loaded_shard_id)
            return
        bn, _ = self._block(param)
        off = 0
        for part, full in enumerate(self.output_sizes):
            rows = _ceil_div(full, bn)
            self._load_part(param, loaded_weight.narrow(0, off, rows), part)
            off += rows

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
    """Query heads are split over the ranks; so are the key/value heads while there are at least as many of them as
    ranks, beyond that every KV head is held by tp_size / total_num_kv_heads consecutive ranks (linear.py:846-870)."""

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int, total_num_kv_heads: int, **kw):
        from ..distributed import get_tensor_model_parallel_world_size as tp_world
        tp = tp_world()
        self.head_size = head_size
        self.num_kv_head_replicas = 1 if tp <= total_num_kv_heads else divide(tp, total_num_kv_heads)
        # (sizes as ColumnParallelLinear divides them: a replicated KV head counts once per rank that holds it)
        kv = max(total_num_kv_heads, tp) * head_size
        sizes = [total_num_heads * head_size, kv, kv]
        super().__init__(hidden_size, sum(sizes), output_sizes=sizes, **kw)

    def weight_loader(self, param, loaded_weight: torch.Tensor, loaded_shard_id: Optional[str] = None) -> None:
        """`loaded_shard_id` "q" / "k" / "v" (linear.py:1035-1195): the checkpoint's q_proj, k_proj or v_proj."""
        if loaded_shard_id is None:
            raise NotImplementedError("QKV weights stored fused on disk are not on this path; pass \"q\", \"k\" or \"v\"")
        part = {"q": 0, "k": 1, "v": 2}[loaded_shard_id]
        src = self.tp_rank if part == 0 else self.tp_rank // self.num_kv_head_replicas
        self._load_part(param, loaded_weight, part, src_block=src)

    def load_full_weight(self, weight: torch.Tensor, weight_scale_inv: torch.Tensor, block: int = 128) -> None:
        """A full [q; k; v] weight (rows of the checkpoint's three projections one after the other) and its scales."""
        q = self.output_sizes[0]
        kv = self.output_sizes[1] // self.num_kv_head_replicas
        assert weight.shape[0] == q + 2 * kv and q % block == 0 and kv % block == 0
        for name, lo, n in (("q", 0, q), ("k", q, kv), ("v", q + kv, kv)):
            self.weight_loader(self.weight, weight[lo : lo + n], name)
            self.weight_loader(self.weight_scale_inv, weight_scale_inv[lo // block : (lo + n) // block], name)


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
        self._attach_loaders()

    def weight_loader(self, param, loaded_weight: torch.Tensor) -> None:
        """This rank's input columns of the full tensor (linear.py:1314-1352); K/128 columns for a scale parameter."""
        _, bk = self._block(param)
        size = _ceil_div(self.input_size_per_partition, bk)
        src = loaded_weight.narrow(1, self.tp_rank * size, size) if self.tp_size > 1 else loaded_weight
        _copy_checked(param.data, src, self.prefix)

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
