"""Standard (no all-to-all) dispatcher, after python/sglang/srt/layers/moe/token_dispatcher/standard.py.

Every rank sees every token; ids of experts owned by other ranks become -1 (:141-173), the MoE
kernels emit zeros for them, and the partial outputs are summed by the tensor-parallel all-reduce in
the layer (`FusedMoE.forward`, fused_moe_triton/layer.py:908-909)."""
from __future__ import annotations

from typing import NamedTuple, Optional

import torch


class StandardTopKOutput(NamedTuple):
    topk_weights: torch.Tensor
    topk_ids: torch.Tensor
    router_logits: Optional[torch.Tensor] = None


class StandardDispatchOutput(NamedTuple):
    hidden_states: torch.Tensor
    hidden_states_scale: Optional[torch.Tensor]
    topk_output: StandardTopKOutput


class StandardCombineInput(NamedTuple):
    hidden_states: torch.Tensor


class StandardDispatcher:
    def __init__(self, num_experts: int, ep_size: int = 1, ep_rank: int = 0):
        self.num_experts = num_experts
        self.ep_size = ep_size
        self.ep_rank = ep_rank
        self.num_local_experts = num_experts // ep_size
        self.local_expert_mapping = None

    def dispatch(self, hidden_states: torch.Tensor, topk_output: StandardTopKOutput) -> StandardDispatchOutput:
        if self.ep_size > 1:
            if self.local_expert_mapping is None:
                m = torch.full((self.num_experts,), -1, dtype=torch.int32, device=hidden_states.device)
                lo = self.ep_rank * self.num_local_experts
                m[lo : lo + self.num_local_experts] = torch.arange(
                    self.num_local_experts, dtype=torch.int32, device=hidden_states.device)
                self.local_expert_mapping = m
            ids = self.local_expert_mapping[topk_output.topk_ids.long()]
            topk_output = StandardTopKOutput(topk_output.topk_weights, ids, topk_output.router_logits)
        return StandardDispatchOutput(hidden_states, None, topk_output)

    def combine(self, combine_input: StandardCombineInput) -> torch.Tensor:
        return combine_input.hidden_states
