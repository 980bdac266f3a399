from .expert_location import ExpertLocationMetadata, topk_ids_logical_to_physical

__all__ = ["ExpertLocationMetadata", "topk_ids_logical_to_physical"]
