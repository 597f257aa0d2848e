"""What a mixer asks of the cache.  A mixer returns one of these from ``cache_need()`` (or None);
layers whose needs are equal share one group of storage, layers with different needs get groups
of their own.

The reference has one kind only: every layer keeps all keys and values of width
n_kv_heads * head_dim (crates/xrt-runtime/src/kv_cache.rs:4-56, crates/xrt-runtime/src/session.rs:46-56).
"""
from __future__ import annotations

from dataclasses import dataclass

BLOCK_TOKENS = 64  # token positions of one cache block; the attention kernels' key tile (csrc/common.cuh)


@dataclass(frozen=True)
class KVNeed:
    """Keys and values indexed by position: [kv head][position][head_dim] for each sequence.
    ``window`` = None keeps every position; a number keeps that many most recent positions
    visible (the storage of a windowed group is its own, so it can be sized and released apart
    from the groups that keep everything)."""
    n_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """A state of fixed size per sequence and layer, zero when a slot is opened."""
    shape: tuple
    dtype: str = "float32"
