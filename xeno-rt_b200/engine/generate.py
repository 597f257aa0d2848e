"""The generation loop: batches of unequal prompts, stop tokens, sequences that end earlier, and
as many batches one after another as there are requests.

The order of decisions for each sequence is the reference's (crates/xrt-runtime/src/session.rs:115-141):
sample from the current logits; a stop id ends the sequence and is neither kept nor emitted
(117-119); a full context ends it (120-122); otherwise the token is appended, counted and reported
(124-129) and fed to the next step (136-141).  Unlike the reference no forward pass runs after the last
token, and the n-gram drafting of session.rs:131-193 is not part of this library.

The loop talks to a *backend* with five methods, so that its decisions can be tested without a
GPU: ``open_slot()``, ``close_slot(slot)``, ``begin(slots, requests)``,
``forward(slots, token_lists) -> logits handle`` (the logits of each sequence's last token), and
``sample(logits, slots, requests) -> list[int]``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from ..cache.spec import BLOCK_TOKENS
from ..core import RuntimeFault
from ..sampling import SamplerConfig


@dataclass
class GenerateRequest:
    """Fields and defaults of the reference's ``GenerateRequest``
    (crates/xrt-runtime/src/session.rs:13-36), with token ids in place of text and a set of stop ids
    in place of the tokenizer's end-of-sequence id (None = the ids of the model's configuration)."""
    prompt_ids: list
    max_tokens: int = 128
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    repetition_penalty: float = 1.1
    seed: int | None = None
    stop_ids: tuple | None = None

    def sampler_config(self) -> SamplerConfig:
        return SamplerConfig(self.temperature, self.top_k, self.top_p, self.repetition_penalty, self.seed)


@dataclass
class GenerateResult:
    tokens: list
    finish_reason: str  # "stop" | "length" | "context"
    prompt_tokens: int


@dataclass
class GenerateStats:
    """What the reference's command prints (crates/xrt-cli/src/main.rs:109-125)."""
    tokens: int = 0
    seconds: float = 0.0
    prefill_seconds: float = 0.0
    decode_steps: int = 0
    batches: int = 0
    first_tokens: int = 0  # tokens that came from a prompt's step rather than a decode step

    @property
    def decode_tokens_per_second(self) -> float:
        rest = self.seconds - self.prefill_seconds
        return (self.tokens - self.first_tokens) / rest if rest > 0 and self.tokens > self.first_tokens else 0.0

    def line(self) -> str:
        total = self.tokens / self.seconds if self.seconds > 0 else 0.0
        return (f"--- {self.tokens} tokens in {self.seconds:.2f}s | prefill {self.prefill_seconds * 1000:.0f}ms | "
                f"decode {self.decode_tokens_per_second:.2f} tok/s | total {total:.2f} tok/s ---")


class SequenceProgress:
    """The decisions for one sequence; no device work."""

    def __init__(self, request: GenerateRequest, stop_ids, context_length: int):
        self.request = request
        self.stop_ids = frozenset(stop_ids)
        self.context_length = context_length
        self.length = len(request.prompt_ids)  # tokens the sequence holds (prompt + kept)
        self.generated: list[int] = []
        self.finish_reason: str | None = None
        if request.max_tokens <= 0:
            self.finish_reason = "length"

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def goes_on_unless_stopped(self) -> bool:
        """Whether the token that is being sampled now will be fed to another step unless it is a stop
        token: what can be said before the token is known."""
        return (not self.finished and self.length < self.context_length
                and len(self.generated) + 1 < self.request.max_tokens)

    def accept(self, token: int) -> bool:
        """Takes the token sampled from the current logits.  Returns True if the token is kept
        and must be fed to the next step, False if the sequence has ended."""
        if self.finished:
            raise RuntimeFault("a finished sequence was given another token")
        if token in self.stop_ids:
            self.finish_reason = "stop"
            return False
        if self.length >= self.context_length:
            self.finish_reason = "context"
            return False
        self.generated.append(token)
        self.length += 1
        if len(self.generated) >= self.request.max_tokens:
            self.finish_reason = "length"
            return False
        return True


def validate_request(request: GenerateRequest, vocab_size: int, context_length: int) -> None:
    """Empty prompts and prompts beyond the context are errors (session.rs:78-93)."""
    if len(request.prompt_ids) == 0:
        raise RuntimeFault("empty prompt: there is no tokenizer here to supply a first token")
    if len(request.prompt_ids) > context_length:
        raise RuntimeFault(f"prompt length {len(request.prompt_ids)} exceeds model context length {context_length}")
    for t in request.prompt_ids:
        if not (0 <= int(t) < vocab_size):
            raise RuntimeFault(f"token id {t} is outside the vocabulary of {vocab_size}")
    request.sampler_config().validate()


def tokens_held(request: GenerateRequest, context_length: int, unit: int = BLOCK_TOKENS) -> int:
    """Cache tokens a request may come to hold, rounded up to the cache's unit."""
    most = min(len(request.prompt_ids) + max(request.max_tokens, 0), context_length)
    return (most + unit - 1) // unit * unit


def plan_batches(requests, context_length: int, capacity_tokens: int, max_batch: int, unit: int = BLOCK_TOKENS):
    """Cuts the requests, in order, into batches that fit the cache: at most ``max_batch``
    sequences and at most ``capacity_tokens`` held tokens a batch.  Returns lists of indices."""
    batches, current, used = [], [], 0
    for i, r in enumerate(requests):
        need = tokens_held(r, context_length, unit)
        if need > capacity_tokens:
            raise RuntimeFault(f"request {i} may hold {need} tokens, the cache holds {capacity_tokens}")
        if current and (len(current) >= max_batch or used + need > capacity_tokens):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += need
    if current:
        batches.append(current)
    return batches


def generate(backend, requests, vocab_size: int, context_length: int, default_stop_ids=(),
             capacity_tokens: int | None = None, max_batch: int = 64, on_token=None):
    """Runs every request to its end, batch after batch.  Returns (results in request order,
    GenerateStats).  ``on_token(request index, token)`` is called for each kept token.

    A backend may offer ``sample_begin`` / ``sample_end`` / ``forward_sampled`` / ``rows``: then the
    next step is started before this step's ids have reached the host (the ids go from the sampler
    to the step on the device), whenever no sequence is about to end for a reason known in advance
    (token limit, context).  A sequence that then ends on a stop token has run one step for nothing;
    the rows of the others are what they would have been.  Decisions and results are the same
    either way."""
    for r in requests:
        validate_request(r, vocab_size, context_length)
    capacity = capacity_tokens if capacity_tokens is not None else sum(
        tokens_held(r, context_length) for r in requests)
    stats = GenerateStats()
    results: list = [None] * len(requests)
    began = time.perf_counter()
    for batch in plan_batches(requests, context_length, capacity, max_batch):
        stats.batches += 1
        progress = {i: SequenceProgress(requests[i], default_stop_ids if requests[i].stop_ids is None
                                        else requests[i].stop_ids, context_length) for i in batch}
        live = [i for i in batch if not progress[i].finished]
        slots = {i: backend.open_slot() for i in live}
        try:
            if live:
                backend.begin([slots[i] for i in live], [requests[i] for i in live])
                t0 = time.perf_counter()
                logits = backend.forward([slots[i] for i in live], [list(requests[i].prompt_ids) for i in live])
                first = True
                pipelined = hasattr(backend, "sample_begin")
                while live:
                    ahead = None
                    if pipelined:
                        pending = backend.sample_begin(logits, [slots[i] for i in live], [requests[i] for i in live])
                        if all(progress[i].goes_on_unless_stopped() for i in live):
                            ahead = backend.forward_sampled([slots[i] for i in live], pending)
                        sampled = backend.sample_end(pending)
                    else:
                        sampled = backend.sample(logits, [slots[i] for i in live], [requests[i] for i in live])
                    if first:
                        stats.prefill_seconds += time.perf_counter() - t0
                        first = False
                    feed, kept_rows = [], []
                    for row, (i, token) in enumerate(zip(live, sampled)):
                        n_before = len(progress[i].generated)
                        keep = progress[i].accept(int(token))
                        if len(progress[i].generated) > n_before:
                            stats.tokens += 1
                            if n_before == 0:
                                stats.first_tokens += 1
                            if on_token is not None:
                                on_token(i, int(token))
                        if keep:
                            feed.append((i, int(token)))
                            kept_rows.append(row)
                        else:
                            backend.close_slot(slots.pop(i))
                    n_before = len(live)
                    live = [i for i, _ in feed]
                    if live:
                        if ahead is None:
                            logits = backend.forward([slots[i] for i in live], [[t] for _, t in feed])
                        else:  # the step is running already; rows of sequences that stopped are dropped
                            logits = ahead if len(live) == n_before else backend.rows(ahead, kept_rows)
                        stats.decode_steps += 1
        finally:
            for slot in slots.values():
                backend.close_slot(slot)
        for i in batch:
            results[i] = GenerateResult(progress[i].generated, progress[i].finish_reason, len(requests[i].prompt_ids))
    stats.seconds = time.perf_counter() - began
    return results, stats
