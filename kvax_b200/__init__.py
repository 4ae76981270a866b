"""kvax_b200: the attention hot path of kvax (block-mask builder, document-masked GQA
flash attention forward/backward, context-parallel token permutation) as hand-written
sm_100a CUDA kernels behind the reference's Python API."""
__version_info__ = (0, 2, 0)
__version__ = ".".join(str(v) for v in __version_info__)

import kvax_b200.ops as ops
import kvax_b200.utils as utils
from kvax_b200.ops import (
    calculate_mask_sparsity,
    check_last_status,
    create_attention_mask,
    flash_attention,
    get_backward_mode,
    get_context_parallel_mode,
    get_context_parallel_overlap,
    get_forward_kernel,
    get_fp32_operand_dtype,
    get_head_exchange_transport,
    last_status,
    print_mask,
    set_backward_mode,
    set_context_parallel_mode,
    set_context_parallel_overlap,
    set_forward_kernel,
    set_fp32_operand_dtype,
    set_head_exchange_transport,
)
from kvax_b200.utils import (
    PADDING_SEGMENT_ID,
    FlashAttentionParamsConfig,
    Mesh,
    attention_specs,
    permute_tokens_context_parallelism,
    unpermute_tokens_context_parallelism,
)

__all__ = list(ops.__all__) + list(utils.__all__)
