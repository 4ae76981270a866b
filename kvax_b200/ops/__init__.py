from kvax_b200._status import check_last_status, last_status
from kvax_b200.ops.flash_attention import (
    flash_attention,
    get_backward_mode,
    get_context_parallel_mode,
    get_context_parallel_overlap,
    get_forward_kernel,
    get_fp32_operand_dtype,
    get_head_exchange_transport,
    set_backward_mode,
    set_context_parallel_mode,
    set_context_parallel_overlap,
    set_forward_kernel,
    set_fp32_operand_dtype,
    set_head_exchange_transport,
)
from kvax_b200.ops.mask_creator import calculate_mask_sparsity, create_attention_mask, print_mask

__all__ = ["flash_attention", "create_attention_mask", "calculate_mask_sparsity", "print_mask",
           "set_context_parallel_mode", "get_context_parallel_mode", "set_context_parallel_overlap",
           "get_context_parallel_overlap", "set_backward_mode", "get_backward_mode",
           "set_head_exchange_transport", "get_head_exchange_transport", "set_fp32_operand_dtype",
           "get_fp32_operand_dtype", "set_forward_kernel", "get_forward_kernel",
           "check_last_status", "last_status"]
