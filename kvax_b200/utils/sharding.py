"""Device mesh for one-process-per-GPU execution and the lookups the ops need.

The reference runs single-controller JAX: a `jax.sharding.Mesh` names device axes and
`shard_map` hands every device its slice (kvax/utils/sharding.py:15-86).  Here every
process owns one GPU and already holds its slice, so the mesh only has to say how many
ranks share each named axis, which coordinate this process has, and which
torch.distributed group spans the context-parallel axis.
"""
from __future__ import annotations

import threading
from typing import Sequence

from kvax_b200.utils.specs import Axes, get_attention_specs

_local = threading.local()


class Mesh:
    """Named axes over the ranks of a torch.distributed job (row-major rank order).

    `Mesh(("data", "context"), (1, 8))`: 8 ranks along "context".  With a single process
    (no process group) every axis must have size 1 unless `rank` is given explicitly,
    which lets host-side logic be exercised without a distributed job."""

    def __init__(self, axis_names: Sequence[str], shape: Sequence[int], rank: int | None = None,
                 groups: dict | None = None):
        if len(axis_names) != len(shape):
            raise ValueError("axis_names and shape must have the same length")
        self.axis_names = tuple(axis_names)
        self.shape = dict(zip(self.axis_names, (int(s) for s in shape)))
        self.size = 1
        for s in shape:
            self.size *= int(s)
        if rank is None:
            rank = 0
            try:
                import torch.distributed as dist
                if dist.is_available() and dist.is_initialized():
                    rank = dist.get_rank()
                    if dist.get_world_size() != self.size:
                        raise ValueError(f"mesh has {self.size} ranks, the job has {dist.get_world_size()}")
            except ImportError:  # pragma: no cover
                pass
        self.rank = rank
        self._groups = dict(groups or {})

    def coordinate(self, axis: str) -> int:
        """Index of this process along `axis`."""
        idx = self.rank
        coord = 0
        for name in reversed(self.axis_names):
            n = self.shape[name]
            if name == axis:
                coord = idx % n
            idx //= n
        return coord

    def group(self, axis: str):
        """torch.distributed group of the ranks that differ only along `axis` (None when
        the axis spans the whole job or has size 1)."""
        if axis in self._groups:
            return self._groups[axis]
        if self.shape[axis] == 1 or self.shape[axis] == self.size:
            return None
        import torch.distributed as dist
        # ranks that share every other coordinate; every process must create all groups
        stride = 1
        for name in reversed(self.axis_names):
            if name == axis:
                break
            stride *= self.shape[name]
        n = self.shape[axis]
        mine = None
        seen = set()
        for r in range(self.size):
            base = r - ((r // stride) % n) * stride
            if base in seen:
                continue
            seen.add(base)
            ranks = [base + i * stride for i in range(n)]
            g = dist.new_group(ranks)
            if self.rank in ranks:
                mine = g
        self._groups[axis] = mine
        return mine

    def __enter__(self):
        stack = getattr(_local, "stack", None)
        if stack is None:
            stack = _local.stack = []
        stack.append(self)
        return self

    def __exit__(self, *exc):
        _local.stack.pop()
        return False


def _get_global_mesh() -> Mesh | None:
    stack = getattr(_local, "stack", None)
    return stack[-1] if stack else None


def _check_mesh_or_get_global(mesh: Mesh | None) -> Mesh:
    if mesh is None:
        mesh = _get_global_mesh()
    if mesh is None:
        raise ValueError(
            "Mesh weren't provided. Either mesh should not be None or global Mesh needs to be set as a context.")
    return mesh


def get_query_context_mesh_axis_name(mesh: Mesh | None) -> str | None:
    """Name of the mesh axis the query sequence is sharded over (None: no context
    parallelism)."""
    _check_mesh_or_get_global(mesh)
    return get_attention_specs().query_specs[Axes.query_sequence]


def get_query_context_mesh_axis_size(mesh: Mesh | None) -> int:
    mesh = _check_mesh_or_get_global(mesh)
    axis = get_query_context_mesh_axis_name(mesh)
    if axis not in mesh.shape:
        raise ValueError(f"Mesh axis {axis} is not present in the device mesh shape.")
    return mesh.shape[axis]
