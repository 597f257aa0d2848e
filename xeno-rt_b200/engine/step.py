"""The step function: a batch of sequences that started together, with unequal lengths; their
prompts in one step, then one token each.  It runs only the tokens it is given, as one batch, from
the cache that earlier steps left, and returns the logits at the wanted places.

The reference has three entry points for one sequence (``forward_token``, ``forward_batch``,
``forward_batch_all_logits``, crates/xrt-models/src/llama.rs:388, 617, 830); here there is one for
many.  Its checks are the reference's (llama.rs:395-408, 434-439, 624-626, 1044-1049): a step continues
exactly where the slot stands, is not empty, and brings ids inside the vocabulary.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import Cache
from ..core import RuntimeFault
from ..parts import StepContext


@dataclass
class StepEntry:
    """One sequence's share of a step: its cache slot, its next tokens, and the places among
    these tokens (0 = the first of them) whose logits are wanted."""
    slot: int
    tokens: list
    want: list = field(default_factory=list)


def build_context(entries, cache: Cache, vocab_size: int, dtype, device, pad_to: int | None = None):
    """Checks the entries, reserves cache room and lays the tokens end to end.  Returns
    (context, wanted rows as a device tensor or None).  ``pad_to`` appends padding rows (slot -1)
    up to that many tokens; padding changes no result."""
    if not entries:
        raise RuntimeFault("a step needs at least one sequence")
    slots = [e.slot for e in entries]
    if len(set(slots)) != len(slots):
        raise RuntimeFault("a slot occurs twice in one step")
    for e in entries:
        if len(e.tokens) == 0:
            raise RuntimeFault(f"slot {e.slot}: a step must bring at least one token")
        lo, hi = min(e.tokens), max(e.tokens)
        if lo < 0 or hi >= vocab_size:
            raise RuntimeFault(f"slot {e.slot}: token id {lo if lo < 0 else hi} is outside the vocabulary of {vocab_size}")
        for w in e.want:
            if not (0 <= w < len(e.tokens)):
                raise RuntimeFault(f"slot {e.slot}: wanted place {w} is outside the {len(e.tokens)} tokens of the step")
    starts = [cache.reserve(e.slot, len(e.tokens)) for e in entries]
    new_lens = [len(e.tokens) for e in entries]
    total = sum(new_lens)
    padded = max(total, pad_to or 0)
    n = len(entries)
    # one int32 buffer, one copy: ids | positions | slots | cu_seqlens | seq_slot | seq_start | wanted rows
    wanted = []
    offset = 0
    buf = np.zeros(3 * padded + (n + 1) + 2 * n, dtype=np.int32)
    ids, pos, slot_of = buf[:padded], buf[padded:2 * padded], buf[2 * padded:3 * padded]
    slot_of[:] = -1
    cu = buf[3 * padded:3 * padded + n + 1]
    seq_slot = buf[3 * padded + n + 1:3 * padded + 2 * n + 1]
    seq_start = buf[3 * padded + 2 * n + 1:]
    for i, e in enumerate(entries):
        k = new_lens[i]
        ids[offset:offset + k] = e.tokens
        pos[offset:offset + k] = np.arange(starts[i], starts[i] + k)
        slot_of[offset:offset + k] = e.slot
        cu[i] = offset
        seq_slot[i] = e.slot
        seq_start[i] = starts[i]
        wanted.extend(offset + w for w in e.want)
        offset += k
    cu[n] = offset
    dev = torch.from_numpy(buf).to(device)
    want_rows = torch.tensor(wanted, dtype=torch.int32, device=device) if wanted else None
    ctx = StepContext(
        n_tokens=padded, n_seqs=n, token_ids=dev[:padded], tok_pos=dev[padded:2 * padded],
        tok_slot=dev[2 * padded:3 * padded], cu_seqlens=dev[3 * padded:3 * padded + n + 1],
        seq_slot=dev[3 * padded + n + 1:3 * padded + 2 * n + 1], seq_start=dev[3 * padded + 2 * n + 1:],
        new_lens=new_lens, starts=starts, all_single=all(k == 1 for k in new_lens), max_new=max(new_lens),
        max_context=max(s + k for s, k in zip(starts, new_lens)), dtype=dtype)
    return ctx, want_rows


class Engine:
    """A model with its cache.  ``step`` is the one way tokens go through the model; generation
    and trace replay both call it."""

    def __init__(self, model, max_tokens: int, max_slots: int | None = None):
        self.model = model
        self.cache = model.new_cache(max_tokens, max_slots)
        self.last_context = None

    def open_slot(self) -> int:
        return self.cache.open_slot()

    def close_slot(self, slot: int) -> None:
        self.cache.close_slot(slot)

    def step(self, entries, pad_to: int | None = None):
        """Runs one step.  ``entries``: StepEntry list.  Returns float32 logits
        [number of wanted places, vocabulary] on the device, in the order of the entries and of
        their ``want`` lists, or None if nothing is wanted."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        model = self.model
        ctx, want_rows = build_context(entries, self.cache, model.vocab_size, model.dtype, model.device, pad_to)
        self.cache.flush_tables()
        self.last_context = ctx
        logits = model.forward(ctx, self.cache, want_rows)
        for e in entries:
            self.cache.advance(e.slot, len(e.tokens))
        return logits
