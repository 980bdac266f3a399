from .weight_utils import load_block_fp8_weights, safetensors_weights_iterator  # noqa: F401
