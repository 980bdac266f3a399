"""Routing that feeds the MoE path.

After python/sglang/srt/layers/moe/topk.py: `fused_topk` (:459-489, `topk_softmax` kernel),
`fused_topk_torch_native` (:427-456) and `biased_grouped_topk_gpu` / `biased_grouped_topk_impl`
(:741-850, :665-738; `moe_fused_gate` kernel).  Inputs are CUDA tensors and go through this library's routing
kernels; there is no CPU form.  The one torch expression left is the reference's own native form of the grouped
routing WITHOUT renormalisation, which its fused kernel does not cover either (:741-850 falls back to it).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def _need_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what}: gating_output must be a CUDA tensor (this path has no CPU implementation)")


def fused_topk(gating_output: torch.Tensor, topk: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    from .... import ops

    _need_cuda(gating_output, "fused_topk")
    g = gating_output.contiguous()
    w = torch.empty(g.shape[0], topk, dtype=torch.float32, device=g.device)
    ids = torch.empty(g.shape[0], topk, dtype=torch.int32, device=g.device)
    ops.topk_softmax_out(w, ids, g, renormalize)
    return w, ids


def biased_grouped_topk(
    gating_output: torch.Tensor, correction_bias: Optional[torch.Tensor], topk: int, renormalize: bool,
    num_expert_group: int, topk_group: int, routed_scaling_factor: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """`routed_scaling_factor` not None = scale the weights by it (apply_routed_scaling_factor_on_output)."""
    _need_cuda(gating_output, "biased_grouped_topk")
    if renormalize:
        from .... import ops

        g = gating_output.contiguous()
        bias = torch.zeros(g.shape[1], dtype=g.dtype, device=g.device) if correction_bias is None \
            else correction_bias.to(g.dtype).contiguous()
        return ops.moe_fused_gate(g, bias, num_expert_group, topk_group, topk, 0,
                                  0.0 if routed_scaling_factor is None else routed_scaling_factor,
                                  routed_scaling_factor is not None)
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
