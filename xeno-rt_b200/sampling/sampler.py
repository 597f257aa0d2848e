"""The sampler: per-sequence state in the cache's state area and one kernel launch a step.

The reference's ``Sampler`` owns a generator and a scratch set of seen ids for ONE sequence
(crates/xrt-runtime/src/sampler.rs:27-48).  Here the state of every live sequence lives beside the
cache, indexed by slot: the key and counter of its random stream and a bitmap of the ids it has
seen; a slot's state is zeroed when the slot is opened.  The stream of a sequence depends only on
its own seed, so what it samples does not depend on what else is in the batch.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..cache import Cache
from ..csrc import ops
from ..weights.random_init import _splitmix64_int
from .params import SamplerConfig

_MASK = (1 << 64) - 1


def sequence_key(seed: int) -> int:
    """The 64-bit key of a sequence's random stream; draw number c (from 0) of the stream is the
    top 32 bits of splitmix64(key + (c + 1) * 0x9E3779B97F4A7C15), divided by 2^32."""
    return _splitmix64_int(seed & _MASK)


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")


class Sampler:
    def __init__(self, cache: Cache, vocab_size: int):
        self.vocab_size = vocab_size
        self.device = cache.device
        words = (vocab_size + 31) // 32
        self.rng_key = cache.register_sequence_state("sampler.rng_key", (), torch.int64)
        self.rng_counter = cache.register_sequence_state("sampler.rng_counter", (), torch.int32)
        self.seen = cache.register_sequence_state("sampler.seen", (words,), torch.int32)
        self._options_key = None
        self._options = None

    def begin(self, slots: list, seeds: list) -> None:
        """Sets the random stream of freshly opened slots (their counters and bitmaps are zero)."""
        keys = np.array([sequence_key(s) for s in seeds], dtype=np.uint64).view(np.int64)
        idx = torch.tensor(slots, dtype=torch.int64, device=self.device)
        self.rng_key.index_copy_(0, idx, torch.from_numpy(keys).to(self.device))

    def observe(self, slots: torch.Tensor, ids: torch.Tensor) -> None:
        """Adds ids[i] to the history of slots[i] (int32 device tensors; slot -1 is skipped)."""
        ops.mark_seen(self.seen, slots, ids, self.vocab_size)

    def sample(self, logits: torch.Tensor, row_slot: torch.Tensor, configs: list) -> torch.Tensor:
        """One id for each row of float32 logits [n, vocab]; ``configs[i]`` are the options of row i.
        Returns an int32 device tensor [n]."""
        n = logits.shape[0]
        key = tuple((c.temperature, c.top_k, c.top_p, c.repetition_penalty) for c in configs)
        if key != self._options_key:  # the options of a batch stay the same from step to step: one copy a batch
            params = np.empty((4, n), dtype=np.float32)
            for i, c in enumerate(configs):
                params[0, i] = c.temperature
                params[1, i] = np.int32(c.top_k).view(np.float32)
                params[2, i] = c.top_p
                params[3, i] = c.repetition_penalty
            self._options = torch.from_numpy(params).to(self.device)
            self._options_key = key
        dev = self._options
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        ops.sample(out, logits, row_slot, dev[0], dev[1].view(torch.int32), dev[2], dev[3], self.seen,
                   self.rng_key, self.rng_counter)
        return out
