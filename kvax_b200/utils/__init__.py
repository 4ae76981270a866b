from kvax_b200.utils.common import PADDING_SEGMENT_ID, FlashAttentionParamsConfig
from kvax_b200.utils.permutation import (
    permute_tokens_context_parallelism,
    unpermute_tokens_context_parallelism,
)
from kvax_b200.utils.sharding import Mesh
from kvax_b200.utils.specs import attention_specs

__all__ = [
    "FlashAttentionParamsConfig",
    "PADDING_SEGMENT_ID",
    "attention_specs",
    "permute_tokens_context_parallelism",
    "unpermute_tokens_context_parallelism",
    "Mesh",
]
