"""B200-native dynamic sparse prefill attention with the operator and patch API of MInference."""
from .configs.model2path import get_support_models
from .minference_configuration import MInferenceConfig
from .models_patch import MInference
from .ops.block_sparse_flash_attention import block_sparse_attention
from .ops.pit_sparse_flash_attention_v2 import vertical_slash_sparse_attention
from .ops.streaming_kernel import streaming_forward
from .patch import patch_hf

__version__ = "0.1.0"

__all__ = [
    "MInference",
    "MInferenceConfig",
    "patch_hf",
    "vertical_slash_sparse_attention",
    "block_sparse_attention",
    "streaming_forward",
    "get_support_models",
]
