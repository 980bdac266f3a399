"""Process groups for the tensor-parallel and expert-parallel forms of the path.

One process per GPU; `torch.distributed` (NCCL on GPUs, gloo in CPU tests) is the transport.
After python/sglang/srt/distributed/parallel_state.py: `GroupCoordinator` (:213), `all_reduce`
(:544-623), `_TP` / `_MOE_EP` (:1392-1429), `communication_op.py:11`.  The reference chooses among
six all-reduce back ends; on one NVSwitch node NCCL (ring or in-switch reduction, its choice) is the
single back end here.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class GroupCoordinator:
    """A set of ranks that communicate; wraps one torch ProcessGroup."""

    def __init__(self, ranks: List[int], backend: Optional[str] = None):
        self.ranks = list(ranks)
        self.world_size = len(self.ranks)
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.rank_in_group = self.ranks.index(self.rank) if self.rank in self.ranks else -1
        if self.world_size > 1:
            self.device_group = dist.new_group(self.ranks, backend=backend)
        else:
            self.device_group = None

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """In-place sum over the group (returns `x`); a no-op for a single rank (:544-549)."""
        if self.world_size == 1:
            return x
        dist.all_reduce(x, group=self.device_group)
        return x

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.world_size == 1:
            return x
        if x.is_cuda and dim % x.dim() == 0:  # rows: one collective straight into the result
            out = torch.empty((self.world_size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(out, x.contiguous(), group=self.device_group)
            return out
        parts = [torch.empty_like(x) for _ in range(self.world_size)]
        dist.all_gather(parts, x.contiguous(), group=self.device_group)
        return torch.cat(parts, dim=dim)

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over the group of `x` [world * n, ...]; this rank keeps rows [rank * n, (rank + 1) * n)."""
        if self.world_size == 1:
            return x
        n = x.shape[0] // self.world_size
        if x.is_cuda:
            out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(out, x.contiguous(), group=self.device_group)
            return out
        x = x.clone()  # (gloo has no reduce-scatter)
        dist.all_reduce(x, group=self.device_group)
        return x[self.rank_in_group * n : (self.rank_in_group + 1) * n].contiguous()

    def all_to_all_single(self, out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits) -> torch.Tensor:
        """Variable-size row exchange: rank r sends inp rows [sum(in_splits[:i]) ...) to peer i."""
        if self.world_size == 1:
            out.copy_(inp)
            return out
        dist.all_to_all_single(out, inp, output_split_sizes=list(out_splits), input_split_sizes=list(in_splits),
                               group=self.device_group)
        return out

    def barrier(self):
        if self.world_size > 1:
            dist.barrier(group=self.device_group)


_TP: Optional[GroupCoordinator] = None
_MOE_EP: Optional[GroupCoordinator] = None


def initialize_model_parallel(tensor_model_parallel_size: int = 1, expert_model_parallel_size: int = 1,
                              backend: Optional[str] = None) -> None:
    """Both groups span ranks [0, size); this path runs one layer type at a time."""
    global _TP, _MOE_EP
    world = dist.get_world_size() if dist.is_initialized() else 1
    assert tensor_model_parallel_size <= world and expert_model_parallel_size <= world
    _TP = GroupCoordinator(list(range(tensor_model_parallel_size)), backend)
    _MOE_EP = GroupCoordinator(list(range(expert_model_parallel_size)), backend)


def destroy_model_parallel() -> None:
    global _TP, _MOE_EP, _FUSED_ROW
    if _FUSED_ROW is not None:
        _FUSED_ROW.close()
        _FUSED_ROW = None
    _TP = None
    _MOE_EP = None


_FUSED_ROW = None


def enable_fused_row_parallel(max_elems: int, device=None):
    """Row-parallel linears of the tensor-parallel group sum their partial outputs with the GEMM-fused all-reduce
    (`fused_row_parallel.FusedRowParallelComm`) whenever the output has at least 128 x world rows and its
    staging copy (world x rows-per-owner x N) fits `max_elems` elements; other shapes keep the NCCL all-reduce.  Collective: every rank of the
    group calls it, after `initialize_model_parallel`.  Returns the communicator (None for a single rank)."""
    global _FUSED_ROW
    tp = get_tp_group()
    if tp.world_size == 1:
        return None
    from .fused_row_parallel import FusedRowParallelComm

    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    _FUSED_ROW = FusedRowParallelComm(tp.device_group, tp.world_size, tp.rank_in_group, max_elems, device)
    return _FUSED_ROW


def get_fused_row_parallel():
    return _FUSED_ROW


def get_tp_group() -> GroupCoordinator:
    global _TP
    if _TP is None:
        _TP = GroupCoordinator([dist.get_rank() if dist.is_initialized() else 0])
    return _TP


def get_moe_ep_group() -> GroupCoordinator:
    global _MOE_EP
    if _MOE_EP is None:
        _MOE_EP = GroupCoordinator([dist.get_rank() if dist.is_initialized() else 0])
    return _MOE_EP


def get_tensor_model_parallel_world_size() -> int:
    return get_tp_group().world_size


def get_tensor_model_parallel_rank() -> int:
    return max(get_tp_group().rank_in_group, 0)


def get_moe_expert_parallel_world_size() -> int:
    return get_moe_ep_group().world_size


def get_moe_expert_parallel_rank() -> int:
    return max(get_moe_ep_group().rank_in_group, 0)


def tensor_model_parallel_all_reduce(x: torch.Tensor) -> torch.Tensor:
    return get_tp_group().all_reduce(x)
