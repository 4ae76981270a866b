from kvax_b200.ops.flash_attention import flash_attention, get_context_parallel_mode, set_context_parallel_mode
from kvax_b200.ops.mask_creator import create_attention_mask

__all__ = ["flash_attention", "create_attention_mask", "set_context_parallel_mode", "get_context_parallel_mode"]
