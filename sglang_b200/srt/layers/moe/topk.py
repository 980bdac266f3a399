"""Routing used to drive the MoE path (torch ops on the device; not part of the timed kernels).

After python/sglang/srt/layers/moe/topk.py: `fused_topk_torch_native` (:427-456) and
`biased_grouped_topk_impl` (:665-738)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def fused_topk(gating_output: torch.Tensor, topk: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    scores = torch.softmax(gating_output.float(), dim=-1)
    w, ids = torch.topk(scores, topk, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.float(), ids.to(torch.int32)


def biased_grouped_topk(
    gating_output: torch.Tensor, correction_bias: Optional[torch.Tensor], topk: int, renormalize: bool,
    num_expert_group: int, topk_group: int, routed_scaling_factor: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    scores = gating_output.float().sigmoid()
    T, E = scores.shape
    choice = scores if correction_bias is None else scores + correction_bias.float().unsqueeze(0)
    group_scores = choice.view(T, num_expert_group, -1).topk(2, dim=-1)[0].sum(dim=-1)
    group_idx = torch.topk(group_scores, k=topk_group, dim=-1, sorted=False)[1]
    group_mask = torch.zeros_like(group_scores).scatter_(1, group_idx, 1)
    score_mask = group_mask.unsqueeze(-1).expand(T, num_expert_group, E // num_expert_group).reshape(T, E)
    tmp = choice.masked_fill(~score_mask.bool(), float("-inf"))
    ids = torch.topk(tmp, k=topk, dim=-1, sorted=False)[1]
    w = scores.gather(1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    if routed_scaling_factor is not None:
        w = w * routed_scaling_factor
    return w.float(), ids.to(torch.int32)
