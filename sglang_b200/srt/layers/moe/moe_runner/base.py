"""`MoeRunnerConfig` as in python/sglang/srt/layers/moe/moe_runner/base.py:25-45 (fields this path reads)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class MoeRunnerConfig:
    num_experts: Optional[int] = None
    num_local_experts: Optional[int] = None
    hidden_size: Optional[int] = None
    intermediate_size_per_partition: Optional[int] = None
    top_k: Optional[int] = None
    activation: str = "silu"
    is_gated: bool = True
    apply_router_weight_on_input: bool = False
    inplace: bool = True
    no_combine: bool = False
    routed_scaling_factor: Optional[float] = None
