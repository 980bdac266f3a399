"""`FusedMoE`: the caller of `Fp8MoEMethod.apply`, with the two expert-parallel forms.

After python/sglang/srt/layers/moe/fused_moe_triton/layer.py:119-918.  Experts are block-distributed:
rank r of an EP group of size p owns experts [r*E/p, (r+1)*E/p) (:182-185).

* a2a_backend "none"  (reference default): every rank holds all tokens, ids of remote experts become
  -1 in the dispatcher, partial outputs are summed with an all-reduce (:908-909).
* a2a_backend "nccl": tokens stay where they were produced; quantised rows travel to the ranks owning
  their experts in one all-to-all, the results return in a second one and are summed at the source.
  This replaces the DeepEP dispatch/combine of the reference
  (python/sglang/srt/layers/moe/token_dispatcher/deepep.py:449-509) with NCCL over NVLink.
  With `equal_tokens_gather_below = n` a batch of at most n tokens over all ranks (decode-sized; every rank must
  hold the SAME number of tokens, as under the reference's padded data-parallel attention) takes the
  gather form instead: all-gather tokens and routing, local experts on all of them with remote ids masked
  to -1, reduce-scatter of the partial outputs (the reference's dp_gather / dp_scatter around its standard
  dispatcher, python/sglang/srt/layers/dp_attention.py).  It needs no host synchronisation and three small
  collectives, which is what a batch of a few tokens is bound by.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import nn

from ....distributed import get_moe_ep_group
from ....eplb import ExpertLocationMetadata, topk_ids_logical_to_physical
from ..moe_runner.base import MoeRunnerConfig
from ..token_dispatcher import StandardDispatcher, StandardTopKOutput
from .ep_a2a import ep_all_to_all_forward


class FusedMoE(nn.Module):
    def __init__(self, num_experts: int, hidden_size: int, intermediate_size: int, top_k: int,
                 params_dtype: torch.dtype = torch.bfloat16, quant_config=None, prefix: str = "",
                 routed_scaling_factor: Optional[float] = None, a2a_backend: str = "none", inplace: bool = False,
                 device=None, equal_tokens_gather_below: Optional[int] = None,
                 expert_location: Optional[ExpertLocationMetadata] = None):
        """`expert_location`: a placement with redundant copies of hot experts (`srt/eplb`); `num_experts` stays the
        number of LOGICAL experts the router names, the layer holds `num_local_physical_experts` of them and maps the
        routed ids to physical slots before dispatching."""
        super().__init__()
        ep = get_moe_ep_group()
        self.moe_ep_size = ep.world_size
        self.moe_ep_rank = max(ep.rank_in_group, 0)
        assert num_experts % self.moe_ep_size == 0
        self.num_logical_experts = num_experts
        self.expert_location = expert_location
        if expert_location is not None:
            assert expert_location.ep_size == self.moe_ep_size and expert_location.num_logical_experts == num_experts
            num_experts = expert_location.num_physical_experts
        self.num_experts = num_experts
        self.num_local_experts = num_experts // self.moe_ep_size
        self.hidden_size = hidden_size
        self.intermediate_size_per_partition = intermediate_size
        self.top_k = top_k
        self.a2a_backend = a2a_backend
        self.equal_tokens_gather_below = equal_tokens_gather_below
        self.quant_config = quant_config
        self.quant_method = quant_config.get_quant_method(self, prefix=prefix)
        self.quant_method.create_weights(self, self.num_local_experts, hidden_size, intermediate_size, params_dtype,
                                         device=device)
        self.moe_runner_config = MoeRunnerConfig(
            num_experts=num_experts, num_local_experts=self.num_local_experts, hidden_size=hidden_size,
            intermediate_size_per_partition=intermediate_size, top_k=top_k, activation="silu", is_gated=True,
            inplace=inplace, routed_scaling_factor=routed_scaling_factor)
        self.quant_method.create_moe_runner(self, self.moe_runner_config)
        self.dispatcher = StandardDispatcher(num_experts, self.moe_ep_size, self.moe_ep_rank)
        self.prefix = prefix
        for name in ("w13_weight", "w2_weight", "w13_weight_scale_inv", "w2_weight_scale_inv"):
            getattr(self, name).weight_loader = self.weight_loader

    # ---- checkpoint loading (layer.py:575-918) -------------------------------------------------------------------
    @classmethod
    def make_expert_params_mapping(cls, ckpt_gate_proj_name: str, ckpt_down_proj_name: str, ckpt_up_proj_name: str,
                                   num_experts: int) -> List[Tuple[str, str, int, str]]:
        """(parameter-name prefix, checkpoint-name fragment, expert id, shard id) for every expert and projection, in
        the form a model's `load_weights` loop matches names with (layer.py:921-947): the checkpoint's
        `experts.<e>.<gate|up>_proj.` tensors are shards "w1" / "w3" of `experts.w13_*`, `down_proj.` is "w2" of
        `experts.w2_*`."""
        out = []
        for e in range(num_experts):
            for shard_id, ckpt in (("w1", ckpt_gate_proj_name), ("w2", ckpt_down_proj_name), ("w3", ckpt_up_proj_name)):
                target = "experts.w2_" if ckpt == ckpt_down_proj_name else "experts.w13_"
                out.append((target, f"experts.{e}.{ckpt}.", e, shard_id))
        return out

    def local_slots_of(self, expert_id: int) -> List[int]:
        """This rank's slots that hold logical expert `expert_id` (none if another rank owns it; more than one only
        under a placement with redundant copies)."""
        if self.expert_location is not None:
            mine = self.expert_location.local_logical_experts(self.moe_ep_rank).tolist()
            return [j for j, e in enumerate(mine) if e == expert_id]
        j = expert_id - self.moe_ep_rank * self.num_local_experts
        return [j] if 0 <= j < self.num_local_experts else []

    def weight_loader(self, param, loaded_weight: torch.Tensor, weight_name: str, shard_id: str, expert_id: int) -> None:
        """One projection of one expert from the checkpoint into its place (layer.py:575-918, block-FP8 branch):
        gate_proj ("w1") fills rows [0, I) of w13, up_proj ("w3") rows [I, 2I), down_proj ("w2") all of w2; a
        `*_scale_inv` parameter takes the rows counted in 128-row blocks.  Experts of other ranks are skipped."""
        if shard_id not in ("w1", "w2", "w3"):
            raise ValueError(f"shard_id must be ['w1','w2','w3'] but got {shard_id}.")
        is_scale = param is self.w13_weight_scale_inv or param is self.w2_weight_scale_inv
        bn = self.quant_config.weight_block_size[0] if is_scale else 1
        half = (self.intermediate_size_per_partition + bn - 1) // bn
        for slot in self.local_slots_of(expert_id):
            dst = param.data[slot]
            if shard_id != "w2":
                dst = dst.narrow(0, 0 if shard_id == "w1" else half, half)
            if tuple(dst.shape) != tuple(loaded_weight.shape):
                raise ValueError(f"{weight_name}: checkpoint tensor of shape {tuple(loaded_weight.shape)} for a "
                                 f"parameter slice of shape {tuple(dst.shape)}")
            if dst.dtype == torch.float8_e4m3fn:
                if loaded_weight.dtype != torch.float8_e4m3fn:
                    raise ValueError(f"{weight_name}: the layer wants serialized float8_e4m3fn, got {loaded_weight.dtype}")
                dst.view(torch.uint8).copy_(loaded_weight.view(torch.uint8))
            else:
                dst.copy_(loaded_weight)

    def load_full_weights(self, w13, w13_s, w2, w2_s) -> None:
        """Takes this rank's experts out of tensors that hold ALL logical experts."""
        if self.expert_location is not None:
            idx = self.expert_location.local_logical_experts(self.moe_ep_rank).long().to(w13.device)
            pick = lambda t: t.view(torch.uint8).index_select(0, idx).view(t.dtype) if t.dtype == torch.float8_e4m3fn \
                else t.index_select(0, idx)
            self.w13_weight.data.copy_(pick(w13))
            self.w13_weight_scale_inv.data.copy_(pick(w13_s))
            self.w2_weight.data.copy_(pick(w2))
            self.w2_weight_scale_inv.data.copy_(pick(w2_s))
            return
        lo = self.moe_ep_rank * self.num_local_experts
        hi = lo + self.num_local_experts
        self.w13_weight.data.copy_(w13[lo:hi])
        self.w13_weight_scale_inv.data.copy_(w13_s[lo:hi])
        self.w2_weight.data.copy_(w2[lo:hi])
        self.w2_weight_scale_inv.data.copy_(w2_s[lo:hi])

    def forward(self, hidden_states: torch.Tensor, topk_output: StandardTopKOutput) -> torch.Tensor:
        if self.expert_location is not None:  # logical ids -> this rank's choice of physical slots
            topk_output = StandardTopKOutput(topk_output[0], topk_ids_logical_to_physical(topk_output[1], self.expert_location),
                                             topk_output[2])
        if self.a2a_backend == "nccl" and self.moe_ep_size > 1:
            n = self.equal_tokens_gather_below
            if n is not None and hidden_states.shape[0] * self.moe_ep_size <= n:
                return self._forward_gathered(hidden_states, topk_output)
            return ep_all_to_all_forward(self, hidden_states, topk_output)
        dispatch_output = self.dispatcher.dispatch(hidden_states, topk_output)
        combine_input = self.quant_method.apply(self, dispatch_output)
        out = self.dispatcher.combine(combine_input)
        if self.moe_ep_size > 1:
            out = get_moe_ep_group().all_reduce(out)
        return out

    def _forward_gathered(self, hidden_states: torch.Tensor, topk_output: StandardTopKOutput) -> torch.Tensor:
        """Every rank quantises its own tokens once and the codes travel (half the bytes of the bf16 rows, as in the
        quantise-before-send of deepep.py:377-390); the local experts take the gathered (codes, scales) as they are."""
        from ..... import ops as _ops
        from .fused_moe import fused_experts_impl

        g = get_moe_ep_group()
        xq, xs = _ops.per_token_group_quant_fp8(hidden_states, self.quant_config.weight_block_size[1])
        q_all = g.all_gather(xq.view(torch.uint8), dim=0).view(torch.float8_e4m3fn)
        s_all = g.all_gather(xs, dim=0)
        w_all = g.all_gather(topk_output[0].float(), dim=0)
        ids_all = g.all_gather(topk_output[1].to(torch.int32), dim=0)
        local = self.dispatcher.dispatch(q_all, StandardTopKOutput(w_all, ids_all, None)).topk_output
        cfg = self.moe_runner_config
        out_all = fused_experts_impl(
            q_all, self.w13_weight, self.w2_weight, local.topk_weights, local.topk_ids, inplace=False,
            use_fp8_w8a8=True, w1_scale=self.w13_weight_scale_inv, w2_scale=self.w2_weight_scale_inv,
            block_shape=self.quant_config.weight_block_size, routed_scaling_factor=cfg.routed_scaling_factor,
            a1_scale=s_all, out_dtype=hidden_states.dtype, has_filtered_ids=True)
        return g.reduce_scatter(out_all)
