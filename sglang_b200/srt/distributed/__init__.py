from .parallel_state import (
    GroupCoordinator,
    destroy_model_parallel,
    enable_fused_row_parallel,
    get_fused_row_parallel,
    get_moe_ep_group,
    get_moe_expert_parallel_rank,
    get_moe_expert_parallel_world_size,
    get_tensor_model_parallel_rank,
    get_tensor_model_parallel_world_size,
    get_tp_group,
    initialize_model_parallel,
    tensor_model_parallel_all_reduce,
)

__all__ = [
    "GroupCoordinator", "destroy_model_parallel", "enable_fused_row_parallel", "get_fused_row_parallel", "get_moe_ep_group", "get_moe_expert_parallel_rank",
    "get_moe_expert_parallel_world_size", "get_tensor_model_parallel_rank",
    "get_tensor_model_parallel_world_size", "get_tp_group", "initialize_model_parallel",
    "tensor_model_parallel_all_reduce",
]
