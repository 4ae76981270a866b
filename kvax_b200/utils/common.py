"""Constants, tile-size configuration and block padding.

Mirrors kvax/utils/common.py: PADDING_SEGMENT_ID (:9), FlashAttentionParamsConfig
(:13-18), get_default_flash_attention_params (:21-41), pad_to_block_size (:44-74).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

PADDING_SEGMENT_ID = -1


@dataclass(frozen=True)
class FlashAttentionParamsConfig:
    """Block sizes the masks are built with.  `num_warps` / `num_stages` are accepted for
    source compatibility; the sm_100a kernels have a fixed warp-specialised layout and
    always compute on 128 x 128 tiles, whatever block size the masks use."""
    query_block_size: int = 64
    kv_block_size: int = 64
    num_warps: int = 4
    num_stages: int = 3


def get_default_flash_attention_params(backward: bool) -> FlashAttentionParamsConfig:
    """Defaults for the device in use.  The reference keys its defaults on the GPU name
    (H100: forward 128/128, backward q64/kv128; anything else 64/64).  On B200 both
    passes use 128/128 so that mask blocks coincide with the kernels' native tiles."""
    if not torch.cuda.is_available():
        raise ValueError("There is must be at least one GPU.")
    name = torch.cuda.get_device_name(0)
    if "B200" in name or "H100" in name or torch.cuda.get_device_capability(0)[0] >= 9:
        return FlashAttentionParamsConfig(query_block_size=128, kv_block_size=128, num_warps=8, num_stages=3)
    return FlashAttentionParamsConfig()


def pad_to_block_size(
    embeddings: Sequence[torch.Tensor] | None,
    positions: torch.Tensor | None,
    segment_ids: torch.Tensor | None,
    block_size: int,
    pos_fill_value: int,
    transposed_inputs: bool = False,
):
    """Pads the sequence axis up to a multiple of `block_size`: embeddings with zeros,
    positions with `pos_fill_value`, segment ids with PADDING_SEGMENT_ID.  The kernels do
    this padding implicitly (out-of-range TMA rows read as zero, out-of-range tokens are
    masked); the function is kept for callers that used it directly."""
    seq_len = positions.shape[1]
    padded = (seq_len + block_size - 1) // block_size * block_size
    pad_len = padded - seq_len
    if pad_len > 0:
        if embeddings is not None:
            axis = 2 if transposed_inputs else 1
            out = []
            for e in embeddings:
                shape = list(e.shape)
                shape[axis] = pad_len
                out.append(torch.cat([e, e.new_zeros(shape)], dim=axis))
            embeddings = out
        if positions is not None:
            positions = torch.nn.functional.pad(positions, (0, pad_len), value=pos_fill_value)
        if segment_ids is not None:
            segment_ids = torch.nn.functional.pad(segment_ids, (0, pad_len), value=PADDING_SEGMENT_ID)
    return embeddings, positions, segment_ids
