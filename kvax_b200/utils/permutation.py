"""Load-balancing token permutation for context parallelism.

Same contract as kvax/utils/permutation.py:45-116: the sequence axis (axis 1) is cut
into 2*CP chunks and reordered to [0, 2CP-1, 1, 2CP-2, ...] so that contiguous slices
of the permuted sequence give every rank one early and one late chunk of a causal
sequence; `unpermute_...` applies the inverse.  Works on full-sequence tensors (the
reference's global arrays), any dtype and trailing shape, single tensor or tuple.
The data movement is a CUDA gather kernel (kvax_b200_permute_tokens).
"""
from __future__ import annotations

import torch

from kvax_b200 import _lib
from kvax_b200.utils.sharding import Mesh, get_query_context_mesh_axis_size


def generate_shard_indices(num_shards: int, reverse: bool = False) -> list[int]:
    """Chunk order [0, n-1, 1, n-2, ...] or, with reverse=True, its inverse."""
    order = []
    for i in range(num_shards // 2):
        order += [i, num_shards - i - 1]
    if not reverse:
        return order
    inverse = [0] * len(order)
    for dst, src in enumerate(order):
        inverse[src] = dst
    return inverse


def _permute_one(x: torch.Tensor, cp: int, reverse: bool) -> torch.Tensor:
    if not x.is_cuda:
        raise _lib.KvaxB200Error("token permutation runs on the GPU; got a CPU tensor (there is no CPU fallback)")
    if x.dim() < 2:
        raise ValueError("expected at least (batch, sequence) dimensions")
    if x.shape[1] % (2 * cp):
        raise ValueError(f"sequence length {x.shape[1]} is not divisible by 2*CP = {2 * cp}")
    x = x.contiguous()
    out = torch.empty_like(x)
    if x.numel() == 0:
        return out
    row_bytes = x.element_size()
    for d in x.shape[2:]:
        row_bytes *= d
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        rc = _lib.load().kvax_b200_permute_tokens(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], row_bytes,
                                                  cp, int(reverse), stream)
    _lib.check(rc, "kvax_b200_permute_tokens")
    return out


def apply_permutation(inputs, num_shards: int, reverse_permutation: bool):
    if len({tuple(t.shape[:2]) for t in inputs}) > 1:
        raise AssertionError("inputs must share their (batch, sequence) dimensions")
    return [_permute_one(t, num_shards // 2, reverse_permutation) for t in inputs]


def permute_tokens_context_parallelism(inputs, mesh: Mesh | None = None):
    num_shards = 2 * get_query_context_mesh_axis_size(mesh)
    single = isinstance(inputs, torch.Tensor)
    outs = apply_permutation((inputs,) if single else tuple(inputs), num_shards, False)
    return outs[0] if single else outs


def unpermute_tokens_context_parallelism(inputs, mesh: Mesh | None = None):
    num_shards = 2 * get_query_context_mesh_axis_size(mesh)
    single = isinstance(inputs, torch.Tensor)
    outs = apply_permutation((inputs,) if single else tuple(inputs), num_shards, True)
    return outs[0] if single else outs
