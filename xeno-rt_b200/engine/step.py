"""The step function: a batch of sequences that started together, with unequal lengths; their
prompts in one step, then one token each.  It runs only the tokens it is given, as one batch, from
the cache that earlier steps left, and returns the logits at the wanted places.

The reference has three entry points for one sequence (``forward_token``, ``forward_batch``,
``forward_batch_all_logits``, crates/xrt-models/src/llama.rs:388, 617, 830); here there is one for
many.  Its checks are the reference's (llama.rs:395-408, 434-439, 624-626, 1044-1049): a step continues
exactly where the slot stands, is not empty, and brings ids inside the vocabulary.

Steps in which every sequence brings one token are replayed from a CUDA graph: the step's arrays
are copied into fixed device buffers (padded with rows that every kernel skips, up to the next
power of two) and one graph launch runs what would otherwise be hundreds of kernel launches.
"""
from __future__ import annotations

import collections
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import Cache
from ..core import RuntimeFault
from ..core.staging import PinnedRing
from ..csrc import ops
from ..parts import StepContext
from ..parts.context import context_bucket

GRAPH_MAX_BATCH = 256
GRAPH_KEEP = 16  # captured decode steps kept at a time; the one used longest ago goes first


@dataclass
class StepEntry:
    """One sequence's share of a step: its cache slot, its next tokens, and the places among
    these tokens (0 = the first of them) whose logits are wanted."""
    slot: int
    tokens: list
    want: list = field(default_factory=list)


def batch_bucket(n: int) -> int:
    """Rows of the captured decode step that serves ``n`` sequences: a power of two up to 8, a
    multiple of 8 beyond (the rows above ``n`` are padding: slot -1)."""
    return 1 << (n - 1).bit_length() if n <= 8 else (n + 7) // 8 * 8


def _check_entries(entries, vocab_size: int) -> None:
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


def layout(padded: int, n: int):
    """Offsets of the step's arrays inside one int32 buffer:
    ids | positions | slots (each ``padded``) | cu_seqlens (n + 1) | seq_slot (n) | seq_start (n)."""
    a = 3 * padded
    return {"ids": (0, padded), "pos": (padded, 2 * padded), "slot": (2 * padded, a), "cu": (a, a + n + 1),
            "seq_slot": (a + n + 1, a + 2 * n + 1), "seq_start": (a + 2 * n + 1, a + 3 * n + 1), "size": a + 3 * n + 1}


def fill_arrays(buf: np.ndarray, entries, starts, padded: int, n_rows: int):
    """Writes the step's arrays into ``buf`` (see ``layout``; ``n_rows`` >= len(entries) sequence
    rows, the rest being padding) and returns the wanted rows."""
    lay = layout(padded, n_rows)
    buf[:lay["size"]] = 0
    ids, pos, slot_of = (buf[lay[k][0]:lay[k][1]] for k in ("ids", "pos", "slot"))
    cu, seq_slot, seq_start = (buf[lay[k][0]:lay[k][1]] for k in ("cu", "seq_slot", "seq_start"))
    slot_of[:] = -1
    seq_slot[:] = -1
    wanted, offset = [], 0
    for i, e in enumerate(entries):
        k = len(e.tokens)
        ids[offset:offset + k] = e.tokens
        pos[offset:offset + k] = np.arange(starts[i], starts[i] + k)
        slot_of[offset:offset + k] = e.slot
        cu[i] = offset
        seq_slot[i] = e.slot
        seq_start[i] = starts[i]
        wanted.extend(offset + w for w in e.want)
        offset += k
    cu[len(entries):] = offset
    return wanted


def mean_context_of(starts, new_lens, rows: int) -> int:
    """The sequences' lengths after the step, summed and divided by the step's rows (padding rows hold nothing)."""
    return -(-sum(s + k for s, k in zip(starts, new_lens)) // max(1, rows))


def context_from(dev: torch.Tensor, padded: int, n_rows: int, new_lens, starts, dtype, max_context=None, mean_context=None):
    lay = layout(padded, n_rows)
    view = lambda k: dev[lay[k][0]:lay[k][1]]
    return StepContext(
        n_tokens=padded, n_seqs=n_rows, token_ids=view("ids"), tok_pos=view("pos"), tok_slot=view("slot"),
        cu_seqlens=view("cu"), seq_slot=view("seq_slot"), seq_start=view("seq_start"), new_lens=list(new_lens),
        starts=list(starts), all_single=all(k == 1 for k in new_lens), max_new=max(new_lens),
        max_context=max_context if max_context is not None else max(s + k for s, k in zip(starts, new_lens)),
        mean_context=mean_context if mean_context is not None else mean_context_of(starts, new_lens, n_rows),
        dtype=dtype)


def build_context(entries, cache: Cache, vocab_size: int, dtype, device, pad_to: int | None = None, staging=None):
    """Checks the entries, reserves cache room and lays the tokens end to end on the device.
    Returns (context, wanted rows as a device tensor or None).  ``pad_to`` appends padding rows
    (slot -1) up to that many tokens; padding changes no result."""
    _check_entries(entries, vocab_size)
    new_lens = [len(e.tokens) for e in entries]
    starts = cache.reserve_all([e.slot for e in entries], new_lens)
    padded = max(sum(new_lens), pad_to or 0)
    n = len(entries)
    size = layout(padded, n)["size"]
    staging = staging or PinnedRing(device, count=1)
    turn, host = staging.take(size)
    wanted = fill_arrays(host.numpy(), entries, starts, padded, n)
    dev = host.to(device, non_blocking=True)
    staging.copied(turn)
    want_rows = torch.tensor(wanted, dtype=torch.int32, device=device) if wanted else None
    return context_from(dev, padded, n, new_lens, starts, dtype), want_rows


class _DecodeGraph:
    """One captured decode step for up to ``bucket`` sequences."""

    def __init__(self, engine: "Engine", bucket: int, context: int, mean_context: int):
        model, cache = engine.model, engine.cache
        self.bucket = bucket
        self.size = layout(bucket, bucket)["size"]
        self.static = torch.zeros(self.size, dtype=torch.int32, device=model.device)
        lay = layout(bucket, bucket)
        self.static[lay["slot"][0]:lay["slot"][1]] = -1
        self.static[lay["seq_slot"][0]:lay["seq_slot"][1]] = -1
        self.rows = torch.arange(bucket, dtype=torch.int32, device=model.device)
        make = lambda: context_from(self.static, bucket, bucket, [1] * bucket, [0] * bucket, model.dtype,
                                    max_context=context, mean_context=mean_context)
        side = torch.cuda.Stream(device=model.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ctx = make()
            ctx.captured = True
            model.forward(ctx, cache, self.rows)  # warm-up: every kernel and allocation once, eagerly
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        # all graphs of an engine capture into one memory pool: they never run at the same time, so
        # the room of one step's intermediates serves every graph
        with torch.cuda.graph(self.graph, pool=engine.graph_pool):
            ctx = make()
            ctx.captured = True
            self.logits = model.forward(ctx, cache, self.rows)
        self.launches = ops.launch_count() - before


class Engine:
    """A model with its cache.  ``step`` is the one way tokens go through the model; generation
    and trace replay both call it."""

    def __init__(self, model, max_tokens: int, max_slots: int | None = None, use_graphs: bool | None = None,
                 tuning: "ops.Tuning | None" = None):
        """``tuning`` (an ``ops.Tuning``) becomes the process's kernel tuning; ``use_graphs`` None
        follows its ``graphs``."""
        self.model = model
        self.cache = model.new_cache(max_tokens, max_slots)
        self.last_context = None
        self.staging = PinnedRing(model.device)
        if tuning is not None:
            ops.set_tuning(tuning)
        if use_graphs is None:
            use_graphs = ops.tuning().graphs
        self.use_graphs = use_graphs and model.device.type == "cuda" and model.graph_safe
        self._graphs: "collections.OrderedDict[tuple, _DecodeGraph]" = collections.OrderedDict()
        #             (batch bucket, context bucket, mean context bucket) -> graph, least recently used first
        self.graph_pool = torch.cuda.graph_pool_handle() if self.use_graphs else None

    def open_slot(self) -> int:
        return self.cache.open_slot()

    def close_slot(self, slot: int) -> None:
        self.cache.close_slot(slot)

    def check_errors(self) -> None:
        """Reads the device's error flag (a synchronisation): raises if a token id outside the
        vocabulary reached the embedding kernel or a bounded wait inside a kernel ran out."""
        ops.check_error_flag(self.model.device)

    def step(self, entries, pad_to: int | None = None, graph: bool | None = None):
        """Runs one step.  ``entries``: StepEntry list.  Returns float32 logits
        [number of wanted places, vocabulary] on the device, in the order of the entries and of
        their ``want`` lists, or None if nothing is wanted."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        model = self.model
        use_graph = self.use_graphs if graph is None else (graph and self.model.graph_safe)
        if (use_graph and pad_to is None and len(entries) <= GRAPH_MAX_BATCH
                and all(len(e.tokens) == 1 for e in entries)):
            return self._graph_step(entries)
        ctx, want_rows = build_context(entries, self.cache, model.vocab_size, model.dtype, model.device, pad_to,
                                       self.staging)
        self.cache.flush_tables()
        self.last_context = ctx
        logits = model.forward(ctx, self.cache, want_rows)
        for e in entries:
            self.cache.advance(e.slot, len(e.tokens))
        return logits

    def step_sampled(self, slots, ids: torch.Tensor):
        """One decode step of the sequences in ``slots`` whose next tokens are ``ids`` (int32, on the
        device, one a sequence, as a sampler left them): the ids never visit the host, so the step
        can be launched before the host has seen them.  Logits of every row.  Falls back to reading
        the ids when the step cannot be replayed from a graph."""
        n = len(slots)
        if self.use_graphs and n <= GRAPH_MAX_BATCH:
            return self._graph_step([StepEntry(s, [0], [0]) for s in slots], ids_device=ids)
        tokens = ids[:n].tolist()
        return self.step([StepEntry(s, [int(t)], [0]) for s, t in zip(slots, tokens)])

    def _graph_step(self, entries, ids_device=None):
        model = self.model
        _check_entries(entries, model.vocab_size)
        n = len(entries)
        bucket = batch_bucket(n)
        starts = self.cache.reserve_all([e.slot for e in entries], [1] * n)
        # launch shapes follow the longest context and, where lengths are unequal, the mean one (both by
        # powers of two): attention cuts its keys finer when most sequences are far shorter than the longest
        key = (bucket, context_bucket(max(starts) + 1), context_bucket(mean_context_of(starts, [1] * n, bucket)))
        g = self._graphs.get(key)
        if g is None:
            while len(self._graphs) >= GRAPH_KEEP:  # a batch that shrinks while its contexts grow meets many keys
                self._graphs.popitem(last=False)
            self.cache.flush_tables()
            g = self._graphs[key] = _DecodeGraph(self, *key)
        self._graphs.move_to_end(key)
        turn, host = self.staging.take(g.size)
        wanted = fill_arrays(host.numpy(), entries, starts, bucket, bucket)
        g.static.copy_(host, non_blocking=True)
        self.staging.copied(turn)
        if ids_device is not None:  # the ids are the first array of the layout
            g.static[:n].copy_(ids_device[:n], non_blocking=True)
        self.cache.flush_tables()
        self.last_context = context_from(g.static, bucket, bucket, [1] * n, starts, model.dtype)
        g.graph.replay()
        ops.add_launches(g.launches)
        for e in entries:
            self.cache.advance(e.slot, 1)
        if not wanted:
            return None
        if wanted == list(range(n)):
            return g.logits[:n].clone()
        return g.logits[torch.tensor(wanted, dtype=torch.int64, device=model.device)]
