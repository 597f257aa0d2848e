"""The cache of one engine.

* A **slot** for each live sequence: its length, its blocks, its fixed-size state.
* **Block storage** for keys and values: a pool of blocks of 64 token positions for each group of
  layers with the same need; a sequence holds ceil(length / 64) blocks of every group, listed in
  the group's block table; blocks go back to the pool when the slot is closed and are used again.
  A group whose layers see only a window of the most recent keys gives a block back as soon as the
  sequence has moved past it: no later token can see its keys (its table entry becomes -1, and the
  attention kernels start at the block that holds the window's first key).
* **Fixed-size state** per sequence: per layer for mixers that ask for it (``StateNeed``), and per
  sequence for whoever registers some (the sampler keeps its generator state and the set of seen
  token ids here).  State is zeroed when a slot is opened.

The reference keeps one ``PagedKvCache`` per session, that is per sequence, with pages of 32
positions allocated on demand per layer (crates/xrt-runtime/src/kv_cache.rs:4-56, 74-98) and
cleared at the start of each generation (crates/xrt-runtime/src/session.rs:58-61); its
preconditions ``cache.len(layer) == position`` (crates/xrt-models/src/llama.rs:434-439) are the
checks of ``reserve`` here.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..core import CacheError, DType, torch_dtype
from ..core.staging import PinnedRing
from .allocator import BlockAllocator, SlotAllocator
from .spec import BLOCK_TOKENS, KVNeed, StateNeed

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32,
                 "int64": torch.int64}


@dataclass
class KVStore:
    """What an attention-like mixer gets for one layer: its key and value pools
    [blocks, kv heads, 64, head_dim] and the block table [slots, blocks per sequence] of its group."""
    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    need: KVNeed


@dataclass
class StateStore:
    """What a mixer with fixed-size state gets for one layer: a tensor [slots, *shape]."""
    state: torch.Tensor
    need: StateNeed


class _KVGroup:
    def __init__(self, need: KVNeed, entries: list[int], n_blocks: int, max_slots: int, blocks_per_seq: int,
                 dtype, device):
        self.need = need
        self.entries = entries
        self.allocator = BlockAllocator(n_blocks)
        shape = (len(entries), max(n_blocks, 1), need.n_kv_heads, BLOCK_TOKENS, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.table_host = np.full((max_slots, blocks_per_seq), -1, dtype=np.int32)
        self.table = torch.full((max_slots, blocks_per_seq), -1, dtype=torch.int32, device=device)
        self.dirty: set[int] = set()
        self.first_block = [0] * max_slots  # blocks before it were given back (windowed groups)

    def blocks_behind_the_window(self, length: int) -> int:
        """How many leading blocks hold no key that a token at position ``length`` or later sees:
        such a token sees positions > its own - window, so a block is done when its last
        position, 64 b + 63, is <= length - window."""
        if self.need.window is None:
            return 0
        return max(0, (length - int(self.need.window) + 1) // BLOCK_TOKENS)

    def nbytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


def _flatten(need, path=()):
    """(path, need) for every single need inside what a place asks for: a need, None, a list of
    those, or a dict from part names to those."""
    if need is None:
        return
    if isinstance(need, dict):
        for key, inner in need.items():
            yield from _flatten(inner, path + (key,))
    elif isinstance(need, (list, tuple)):
        for i, inner in enumerate(need):
            yield from _flatten(inner, path + (i,))
    else:
        yield path, need


def _rebuild(need, stores: dict, path=()):
    """The stores in the shape in which the needs were given."""
    if need is None:
        return None
    if isinstance(need, dict):
        return {key: _rebuild(inner, stores, path + (key,)) for key, inner in need.items()}
    if isinstance(need, (list, tuple)):
        return [_rebuild(inner, stores, path + (i,)) for i, inner in enumerate(need)]
    return stores[path]


class Cache:
    """See the module text.  ``needs`` has one entry for each place of the model's schedule: what
    the place's parts ask for.  An entry is a ``KVNeed``, a ``StateNeed``, None (a place that owns
    no cache, e.g. because it reads another place's), a list of those (a part that wants several
    storages, say keys and a fixed-size state), or a dict from part names to those (a layer with
    several parts that keep something); ``store(place)`` answers in the same shape."""

    def __init__(self, needs: list, max_tokens: int, max_positions: int, dtype: DType, device,
                 max_slots: int | None = None):
        if max_tokens <= 0:
            raise CacheError(f"max_tokens {max_tokens} must be positive")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_positions = max_positions
        self.n_blocks = (max_tokens + BLOCK_TOKENS - 1) // BLOCK_TOKENS
        self.blocks_per_seq = min(self.n_blocks, (max_positions + BLOCK_TOKENS - 1) // BLOCK_TOKENS)
        self.max_slots = max_slots if max_slots is not None else min(self.n_blocks, 1024)
        if self.max_slots <= 0:
            raise CacheError(f"max_slots {self.max_slots} must be positive")
        self.slots = SlotAllocator(self.max_slots)
        self._table_ring = PinnedRing(self.device)
        self.lengths = [0] * self.max_slots
        self._n_seq_blocks = [0] * self.max_slots

        kv_needs: dict[KVNeed, list] = {}
        state_needs: dict[StateNeed, list] = {}
        self._needs = list(needs)
        for place, asked in enumerate(needs):
            for path, need in _flatten(asked):
                if isinstance(need, KVNeed):
                    kv_needs.setdefault(need, []).append((place, path))
                elif isinstance(need, StateNeed):
                    state_needs.setdefault(need, []).append((place, path))
                else:
                    raise CacheError(f"schedule place {place}: unknown cache need {need!r}")
        tdtype = torch_dtype(dtype)
        self.kv_groups = [_KVGroup(need, entries, self.n_blocks, self.max_slots, self.blocks_per_seq, tdtype,
                                   self.device) for need, entries in kv_needs.items()]
        self.state_groups = []
        for need, entries in state_needs.items():
            if need.dtype not in _STATE_DTYPES:
                raise CacheError(f"state dtype {need.dtype!r} is not one of {sorted(_STATE_DTYPES)}")
            tensor = torch.zeros((len(entries), self.max_slots) + tuple(need.shape),
                                 dtype=_STATE_DTYPES[need.dtype], device=self.device)
            self.state_groups.append((need, entries, tensor))
        flat: dict[int, dict] = {}
        for group in self.kv_groups:
            for i, (place, path) in enumerate(group.entries):
                flat.setdefault(place, {})[path] = KVStore(group.k[i], group.v[i], group.table, group.need)
        for need, entries, tensor in self.state_groups:
            for i, (place, path) in enumerate(entries):
                flat.setdefault(place, {})[path] = StateStore(tensor[i], need)
        self._stores = {place: _rebuild(asked, flat.get(place, {})) for place, asked in enumerate(needs)}
        self.sequence_state: dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ storage
    def store(self, entry: int):
        """The storage of schedule place ``entry``, in the shape in which the place asked for it
        (a KVStore or StateStore, None, a list, or a dict by part name)."""
        return self._stores.get(entry)

    def register_sequence_state(self, name: str, shape: tuple, dtype) -> torch.Tensor:
        """A tensor [slots, *shape] of per-sequence state, zeroed when a slot is opened."""
        if name in self.sequence_state:
            existing = self.sequence_state[name]
            if tuple(existing.shape[1:]) != tuple(shape) or existing.dtype != dtype:
                raise CacheError(f"sequence state {name!r} is registered with another shape or dtype")
            return existing
        tensor = torch.zeros((self.max_slots,) + tuple(shape), dtype=dtype, device=self.device)
        self.sequence_state[name] = tensor
        return tensor

    @property
    def capacity_tokens(self) -> int:
        """Token positions the block pools hold."""
        return self.n_blocks * BLOCK_TOKENS

    def nbytes(self) -> int:
        total = sum(g.nbytes() for g in self.kv_groups)
        total += sum(t.numel() * t.element_size() for _, _, t in self.state_groups)
        total += sum(t.numel() * t.element_size() for t in self.sequence_state.values())
        return total

    # ------------------------------------------------------------------ slots
    def open_slot(self) -> int:
        slot = self.slots.open()
        self.lengths[slot] = 0
        self._n_seq_blocks[slot] = 0
        for _, _, tensor in self.state_groups:
            tensor[:, slot].zero_()
        for tensor in self.sequence_state.values():
            tensor[slot].zero_()
        return slot

    def close_slot(self, slot: int) -> None:
        if not self.slots.is_open(slot):
            raise CacheError(f"slot {slot} is not open (closed twice, or never opened)")
        n = self._n_seq_blocks[slot]
        for group in self.kv_groups:
            group.allocator.give_back(int(b) for b in group.table_host[slot, group.first_block[slot]:n])
            group.table_host[slot, :n] = -1
            group.first_block[slot] = 0
            group.dirty.add(slot)
        self._n_seq_blocks[slot] = 0
        self.lengths[slot] = 0
        self.slots.close(slot)

    def length(self, slot: int) -> int:
        if not self.slots.is_open(slot):
            raise CacheError(f"slot {slot} is not open")
        return self.lengths[slot]

    def reserve(self, slot: int, n_new: int) -> int:
        """Makes room for ``n_new`` more tokens of ``slot`` and returns where they start.  The
        length moves only with ``advance``.  Raises if the slot is not open, the sequence would
        pass the model's positions, or the pool has no block left."""
        start = self.length(slot)
        if n_new <= 0:
            raise CacheError(f"slot {slot}: a step must bring at least one token, got {n_new}")
        if start + n_new > self.max_positions:
            raise CacheError(f"slot {slot}: {start} + {n_new} tokens pass the model's {self.max_positions} positions")
        need_blocks = (start + n_new + BLOCK_TOKENS - 1) // BLOCK_TOKENS
        have = self._n_seq_blocks[slot]
        if need_blocks > self.blocks_per_seq:
            raise CacheError(f"slot {slot}: {need_blocks} blocks pass the {self.blocks_per_seq} a sequence may hold")
        if need_blocks > have:
            extra = need_blocks - have
            for group in self.kv_groups:
                if group.allocator.free < extra:
                    raise CacheError(f"the cache is full: slot {slot} needs {extra} more blocks of {BLOCK_TOKENS} "
                                     f"tokens, {group.allocator.free} of {group.allocator.count} are free")
            for group in self.kv_groups:
                group.table_host[slot, have:need_blocks] = group.allocator.take(extra)
                group.dirty.add(slot)
            self._n_seq_blocks[slot] = need_blocks
        return start

    def unreserve(self, slot: int) -> None:
        """Gives back the blocks that ``reserve`` took for tokens that never came (what the slot
        holds beyond its length)."""
        keep = max((self.length(slot) + BLOCK_TOKENS - 1) // BLOCK_TOKENS, 0)
        have = self._n_seq_blocks[slot]
        if have <= keep:
            return
        for group in self.kv_groups:
            first = max(keep, group.first_block[slot])
            group.allocator.give_back(int(b) for b in group.table_host[slot, first:have])
            group.table_host[slot, keep:have] = -1
            group.dirty.add(slot)
        self._n_seq_blocks[slot] = keep

    def reserve_all(self, slots, counts) -> list:
        """``reserve`` for every sequence of a step, or for none: if one of them cannot be served,
        what the earlier ones just took goes back before the error is raised."""
        starts = []
        try:
            for slot, n_new in zip(slots, counts):
                starts.append(self.reserve(slot, n_new))
        except CacheError:
            for slot in list(slots)[:len(starts)]:
                self.unreserve(slot)
            raise
        return starts

    def advance(self, slot: int, n_new: int) -> None:
        if self.length(slot) + n_new > self._n_seq_blocks[slot] * BLOCK_TOKENS:
            raise CacheError(f"slot {slot}: advancing by {n_new} passes what was reserved")
        self.lengths[slot] += n_new
        for group in self.kv_groups:
            done = min(group.blocks_behind_the_window(self.lengths[slot]), self._n_seq_blocks[slot])
            first = group.first_block[slot]
            if done > first:
                # Kernels already launched still read the old table and the old blocks: the table
                # changes with the next flush and the blocks are written again only by later steps.
                group.allocator.give_back(int(b) for b in group.table_host[slot, first:done])
                group.table_host[slot, first:done] = -1
                group.first_block[slot] = done
                group.dirty.add(slot)

    def flush_tables(self) -> None:
        """Brings the device block tables up to date with the host's (before kernels read them)."""
        for group in self.kv_groups:
            if not group.dirty:
                continue
            rows = sorted(group.dirty)
            if self.device.type == "cuda":
                # the changed rows and their numbers through one pinned buffer and one copy that the host
                # does not wait for: with sequences of unequal lengths some row changes at nearly every step
                width = group.table_host.shape[1]
                turn, host = self._table_ring.take(len(rows) * (width + 1))
                host[:len(rows)] = torch.tensor(rows, dtype=torch.int32)
                host[len(rows):].view(len(rows), width).copy_(torch.from_numpy(group.table_host[rows]))
                dev = host.to(self.device, non_blocking=True)
                self._table_ring.copied(turn)
                group.table.index_copy_(0, dev[:len(rows)].to(torch.int64), dev[len(rows):].view(len(rows), width))
            else:
                group.table[rows] = torch.from_numpy(group.table_host[rows])
            group.dirty.clear()

    # ------------------------------------------------------------------ checks
    def blocks_free(self) -> int:
        return min((g.allocator.free for g in self.kv_groups), default=self.n_blocks)

    def check(self) -> None:
        """Raises if a block is lost or held twice (used by tests)."""
        self.slots.check()
        for group in self.kv_groups:
            group.allocator.check()
            held = []
            for slot in range(self.max_slots):
                row = group.table_host[slot]
                n = self._n_seq_blocks[slot] if self.slots.is_open(slot) else 0
                first = group.first_block[slot] if self.slots.is_open(slot) else 0
                if (row[n:] != -1).any() or (row[:first] != -1).any():
                    raise CacheError(f"slot {slot} lists blocks beyond what it holds")
                if (row[first:n] < 0).any():
                    raise CacheError(f"slot {slot} misses a block that it should hold")
                if first > group.blocks_behind_the_window(self.lengths[slot]):
                    raise CacheError(f"slot {slot} gave back a block that its window still covers")
                held.extend(int(b) for b in row[first:n])
            if len(held) != len(set(held)):
                raise CacheError("a block is listed by two sequences")
            if len(held) != group.allocator.held:
                raise CacheError(f"{group.allocator.held} blocks are held but {len(held)} are listed")
