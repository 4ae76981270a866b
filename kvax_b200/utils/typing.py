"""AttentionMask container (kvax/utils/typing.py:15-37)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

DeviceArray = torch.Tensor
Specs = tuple
FlattenedAttentionMask = tuple


@dataclass
class AttentionMask:
    """Four int32 tensors of shape (batch, 1, n_outer_blocks): for every block of the
    outer axis, the first / one-past-last inner block that may be attended and the first /
    one-past-last inner block that is attended in full."""
    lower_bounds: torch.Tensor
    upper_bounds: torch.Tensor
    lower_full_bounds: torch.Tensor
    upper_full_bounds: torch.Tensor

    def flatten(self) -> FlattenedAttentionMask:
        return (self.lower_bounds, self.upper_bounds, self.lower_full_bounds, self.upper_full_bounds)

    @classmethod
    def unflatten(cls, flatten_mask: FlattenedAttentionMask) -> "AttentionMask":
        return cls(lower_bounds=flatten_mask[0], upper_bounds=flatten_mask[1],
                   lower_full_bounds=flatten_mask[2], upper_full_bounds=flatten_mask[3])
