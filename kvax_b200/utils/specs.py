"""Global registry of the sharding specs of query and key/value tensors.

Same contract as kvax/utils/specs.py:9-112: a module-level (not thread-local) pair of
4-tuples (batch, sequence, heads, head_dim) naming mesh axes or None, validated on
assignment, with a context manager that restores the previous pair on exit.
"""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass
from enum import IntEnum
from typing import Generator


@dataclass
class AttentionSpecs:
    query_specs: tuple | None = None
    kv_specs: tuple | None = None


class Axes(IntEnum):
    batch = 0
    query_sequence = 1
    kv_sequence = 1
    heads = 2
    kv_heads = 2
    head_dim = 3


_attention_specs = AttentionSpecs()


def _validate_attention_specs(query_specs, kv_specs) -> None:
    for name, specs in (("query_specs", query_specs), ("kv_specs", kv_specs)):
        if len(specs) != 4:
            raise ValueError(f"{name} must have exactly 4 dimensions, got {len(specs)}.")
    if query_specs[Axes.batch] != kv_specs[Axes.batch]:
        raise ValueError("Batch dimension sharding must match between query_specs and kv_specs.")
    if query_specs[Axes.head_dim] != kv_specs[Axes.head_dim]:
        raise ValueError("head_dim dimension sharding must match between query_specs and kv_specs.")
    if kv_specs[Axes.kv_sequence] is not None:
        raise ValueError("Context parallelism with sharded key/value tensors is not supported.")
    if kv_specs[Axes.head_dim] is not None:
        raise ValueError("Sharding of attention_head_dim is not supported.")


def set_attention_specs(query_specs, kv_specs) -> None:
    _validate_attention_specs(query_specs, kv_specs)
    _attention_specs.query_specs = query_specs
    _attention_specs.kv_specs = kv_specs


def get_attention_specs() -> AttentionSpecs:
    if _attention_specs.query_specs is None or _attention_specs.kv_specs is None:
        raise ValueError("Attention specifications must be initialised before calling get_attention_specs.")
    return _attention_specs


@contextmanager
def attention_specs(query_specs, kv_specs) -> Generator[None, None, None]:
    previous = (_attention_specs.query_specs, _attention_specs.kv_specs)
    set_attention_specs(query_specs, kv_specs)
    try:
        yield
    finally:
        _attention_specs.query_specs, _attention_specs.kv_specs = previous
