"""Counterpart of python/sglang/srt/layers/moe/fused_moe_triton/moe_align_block_size.py."""
from __future__ import annotations

from typing import Tuple

import torch

from ..... import ops as _ops


def moe_align_block_size(
    topk_ids: torch.Tensor, block_size: int, num_experts: int
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Same contract as the reference wrapper (:17-82): returns (sorted_token_ids, expert_ids,
    num_tokens_post_padded).  Ids may be -1 (expert on another rank); those entries form leading
    blocks with expert id -1.  Unlike the reference kernel the order inside an expert is
    deterministic (ascending flat index)."""
    return _ops.moe_align_block_size(topk_ids, block_size, num_experts)
