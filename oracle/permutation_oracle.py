"""CPU oracle for the context-parallel token permutation.  TEST INFRASTRUCTURE ONLY.

Restates kvax/utils/permutation.py:9-42 in NumPy: the sequence axis (axis 1) is cut
into 2*CP chunks and chunk order becomes [0, 2CP-1, 1, 2CP-2, ...]; the inverse uses
the argsort of that order.  Pure data movement, so results must be bit-exact.
Pinned by the known index lists in the reference's survey probes (CP=2 -> [0,3,1,2])
and by tests/test_oracle_permutation.py.
"""
from __future__ import annotations

import numpy as np


def shard_indices(num_shards: int, reverse: bool = False) -> np.ndarray:
    """permutation.py:9-15"""
    idx = np.array([(i, num_shards - i - 1) for i in range(num_shards // 2)]).flatten()
    return np.argsort(idx) if reverse else idx


def apply_permutation(x: np.ndarray, cp: int, reverse: bool) -> np.ndarray:
    """permutation.py:18-42 for one array."""
    n = 2 * cp
    idx = shard_indices(n, reverse)
    b = x.shape[0]
    return x.reshape(b, n, -1, *x.shape[2:])[:, idx].reshape(x.shape)


def permute(x, cp):
    return apply_permutation(np.asarray(x), cp, False)


def unpermute(x, cp):
    return apply_permutation(np.asarray(x), cp, True)
