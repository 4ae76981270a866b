from kvax_b200.ops.flash_attention import flash_attention
from kvax_b200.ops.mask_creator import create_attention_mask

__all__ = ["flash_attention", "create_attention_mask"]
