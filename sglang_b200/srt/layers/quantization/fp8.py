"""Counterpart of python/sglang/srt/layers/quantization/fp8.py restricted to block-wise FP8.

`Fp8Config` (:108-185), `Fp8LinearMethod` (:188-527) and `Fp8MoEMethod` (:530-1167) keep the
reference's constructor / create_weights / apply signatures and the parameter names and shapes a
DeepSeek-style block-FP8 checkpoint loads into (`weight`, `weight_scale_inv`, `w13_weight`,
`w2_weight`, `w13_weight_scale_inv`, `w2_weight_scale_inv`).  Every `apply` runs the sm_100a kernels;
there is no back-end selection.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch.nn import Module
from torch.nn.parameter import Parameter

from ...distributed import get_tensor_model_parallel_world_size
from ..moe.fused_moe_triton.fused_moe import fused_experts
from ..moe.moe_runner.base import MoeRunnerConfig
from ..moe.token_dispatcher import StandardCombineInput, StandardDispatchOutput
from .fp8_utils import dispatch_w8a8_block_fp8_linear

ACTIVATION_SCHEMES = ["static", "dynamic"]


class Fp8Config:
    """fp8.py:108-185."""

    def __init__(
        self,
        is_checkpoint_fp8_serialized: bool = True,
        activation_scheme: str = "dynamic",
        ignored_layers: Optional[List[str]] = None,
        weight_block_size: Optional[List[int]] = None,
    ) -> None:
        if activation_scheme not in ACTIVATION_SCHEMES:
            raise ValueError(f"Unsupported activation scheme {activation_scheme}")
        if weight_block_size is None:
            weight_block_size = [128, 128]
        if not is_checkpoint_fp8_serialized:
            raise ValueError("The block-wise quantization only supports fp8-serialized checkpoint for now.")
        if len(weight_block_size) != 2:
            raise ValueError(f"The quantization block size of weight must have 2 dimensions, got {len(weight_block_size)}")
        if activation_scheme != "dynamic":
            raise ValueError(f"The block-wise quantization only supports dynamic activation scheme, got {activation_scheme}")
        if list(weight_block_size) != [128, 128]:
            raise ValueError("this implementation supports weight_block_size [128, 128] only")
        self.is_checkpoint_fp8_serialized = is_checkpoint_fp8_serialized
        self.activation_scheme = activation_scheme
        self.ignored_layers = ignored_layers or []
        self.weight_block_size = list(weight_block_size)

    @classmethod
    def get_name(cls) -> str:
        return "fp8"

    @classmethod
    def get_supported_act_dtypes(cls) -> List[torch.dtype]:
        return [torch.bfloat16, torch.half]

    @classmethod
    def get_min_capability(cls) -> int:
        return 100

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "Fp8Config":
        quant_method = config.get("quant_method", "fp8")
        return cls(
            is_checkpoint_fp8_serialized="fp8" in quant_method,
            activation_scheme=config.get("activation_scheme", "dynamic"),
            ignored_layers=config.get("ignored_layers"),
            weight_block_size=config.get("weight_block_size"),
        )

    def get_quant_method(self, layer: Module, prefix: str = ""):
        from ..linear import LinearBase
        from ..moe.fused_moe_triton.layer import FusedMoE

        if isinstance(layer, LinearBase):
            return Fp8LinearMethod(self)
        if isinstance(layer, FusedMoE):
            return Fp8MoEMethod(self)
        return None


class Fp8LinearMethod:
    """fp8.py:188-527, block-quant branch."""

    def __init__(self, quant_config: Fp8Config):
        self.quant_config = quant_config
        self.block_quant = self.quant_config.weight_block_size is not None
        self.w8a8_block_fp8_linear = dispatch_w8a8_block_fp8_linear()

    def create_weights(
        self,
        layer: Module,
        input_size_per_partition: int,
        output_partition_sizes: List[int],
        input_size: int,
        output_size: int,
        params_dtype: torch.dtype,
        **extra_weight_attrs,
    ):
        output_size_per_partition = sum(output_partition_sizes)
        tp_size = get_tensor_model_parallel_world_size()
        block_n, block_k = self.quant_config.weight_block_size
        # divisibility rules of fp8.py:236-259
        if tp_size > 1 and input_size // input_size_per_partition == tp_size:
            if input_size_per_partition % block_k != 0:
                raise ValueError(
                    f"Weight input_size_per_partition = {input_size_per_partition} is not divisible by "
                    f"weight quantization block_k = {block_k}.")
        if (tp_size > 1 and output_size // output_size_per_partition == tp_size) or len(output_partition_sizes) > 1:
            for output_partition_size in output_partition_sizes:
                if output_partition_size % block_n != 0:
                    raise ValueError(
                        f"Weight output_partition_size = {output_partition_size} is not divisible by "
                        f"weight quantization block_n = {block_n}.")
        layer.logical_widths = output_partition_sizes
        layer.input_size_per_partition = input_size_per_partition
        layer.output_size_per_partition = output_size_per_partition
        layer.orig_dtype = params_dtype
        device = extra_weight_attrs.get("device")
        weight = Parameter(
            torch.empty(output_size_per_partition, input_size_per_partition, dtype=torch.float8_e4m3fn, device=device),
            requires_grad=False)
        layer.register_parameter("weight", weight)
        scale = Parameter(
            torch.full(
                ((output_size_per_partition + block_n - 1) // block_n,
                 (input_size_per_partition + block_k - 1) // block_k),
                torch.finfo(torch.float32).min, dtype=torch.float32, device=device),
            requires_grad=False)
        scale.format_ue8m0 = False
        layer.register_parameter("weight_scale_inv", scale)
        layer.register_parameter("input_scale", None)

    def process_weights_after_loading(self, layer: Module) -> None:
        # fp8.py:331-377: nothing to do for float32 block scales on CUDA (no UE8M0 re-quantisation here)
        layer.weight.data = layer.weight.data.contiguous()
        layer.weight_scale_inv.data = layer.weight_scale_inv.data.contiguous()

    def apply(self, layer: Module, x, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp8.py:471-527.  `x` may be a (codes, scales) tuple for pre-quantised input (:500-508)."""
        if isinstance(x, tuple):
            return self.w8a8_block_fp8_linear(
                input=x[0], weight=layer.weight, block_size=self.quant_config.weight_block_size,
                weight_scale=layer.weight_scale_inv, input_scale=x[1], bias=bias)
        return self.w8a8_block_fp8_linear(
            input=x, weight=layer.weight, block_size=self.quant_config.weight_block_size,
            weight_scale=layer.weight_scale_inv, input_scale=None, bias=bias)


class Fp8MoEMethod:
    """fp8.py:530-1167, block-quant branch with the single (B200) runner."""

    def __init__(self, quant_config: Fp8Config):
        self.quant_config = quant_config
        self.block_quant = self.quant_config.weight_block_size is not None
        self.moe_runner_config: Optional[MoeRunnerConfig] = None

    def create_weights(
        self,
        layer: Module,
        num_experts: int,
        hidden_size: int,
        intermediate_size_per_partition: int,
        params_dtype: torch.dtype,
        **extra_weight_attrs,
    ):
        block_n, block_k = self.quant_config.weight_block_size
        tp_size = get_tensor_model_parallel_world_size()
        # fp8.py:567-587
        if intermediate_size_per_partition % block_n != 0:
            raise ValueError(
                f"The output_size of gate's and up's weight = {intermediate_size_per_partition} is not divisible by "
                f"weight quantization block_n = {block_n}.")
        if tp_size > 1 and intermediate_size_per_partition % block_k != 0:
            raise ValueError(
                f"The input_size of down's weight = {intermediate_size_per_partition} is not divisible by "
                f"weight quantization block_k = {block_k}.")
        device = extra_weight_attrs.get("device")
        fp8 = torch.float8_e4m3fn
        layer.register_parameter("w13_weight", Parameter(
            torch.empty(num_experts, 2 * intermediate_size_per_partition, hidden_size, dtype=fp8, device=device),
            requires_grad=False))
        layer.register_parameter("w2_weight", Parameter(
            torch.empty(num_experts, hidden_size, intermediate_size_per_partition, dtype=fp8, device=device),
            requires_grad=False))
        layer.register_parameter("w13_weight_scale_inv", Parameter(
            torch.ones(num_experts, 2 * ((intermediate_size_per_partition + block_n - 1) // block_n),
                       (hidden_size + block_k - 1) // block_k, dtype=torch.float32, device=device),
            requires_grad=False))
        layer.register_parameter("w2_weight_scale_inv", Parameter(
            torch.ones(num_experts, (hidden_size + block_n - 1) // block_n,
                       (intermediate_size_per_partition + block_k - 1) // block_k, dtype=torch.float32, device=device),
            requires_grad=False))
        layer.w13_input_scale = None
        layer.w2_input_scale = None

    def process_weights_after_loading(self, layer: Module) -> None:
        for name in ("w13_weight", "w2_weight", "w13_weight_scale_inv", "w2_weight_scale_inv"):
            p = getattr(layer, name)
            p.data = p.data.contiguous()

    def create_moe_runner(self, layer: Module, moe_runner_config: MoeRunnerConfig):
        self.moe_runner_config = moe_runner_config

    def apply(self, layer: Module, dispatch_output: StandardDispatchOutput) -> StandardCombineInput:
        """fp8.py:1023-1167 -> MoeRunner.run -> fused_experts (moe_runner/triton.py:328-361)."""
        cfg = self.moe_runner_config or MoeRunnerConfig()
        output = fused_experts(
            dispatch_output.hidden_states, layer.w13_weight, layer.w2_weight, dispatch_output.topk_output, cfg,
            w13_scale=layer.w13_weight_scale_inv, w2_scale=layer.w2_weight_scale_inv,
            block_shape=self.quant_config.weight_block_size,
            has_filtered_ids=getattr(layer, "moe_ep_size", 1) > 1)
        return StandardCombineInput(hidden_states=output)
