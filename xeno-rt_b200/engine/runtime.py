"""The Python entry point, in the manner of the reference's runtime crate:
``Runtime.load(path)`` -> ``runtime.new_session()`` -> ``session.generate(request)``
(crates/xrt-runtime/src/lib.rs:15-47, crates/xrt-runtime/src/session.rs:38-69).

A reference session holds one sequence; a session here holds an engine (model + cache + sampler)
and also runs batches of requests.
"""
from __future__ import annotations

import torch

from ..core import RuntimeFault
from ..sampling import Sampler
from ..sampling.sampler import fresh_seed
from .generate import GenerateRequest, generate, tokens_held
from .model import Model
from .step import Engine, StepEntry


class DeviceBackend:
    """The generation loop's backend on the GPU: the engine's step function and the sampler."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.sampler = Sampler(engine.cache, engine.model.vocab_size)
        self.track_seen = True
        self._host = None  # pinned: the step's ids and the error flag
        self._explicit_slots = False

    def open_slot(self) -> int:
        return self.engine.open_slot()

    def close_slot(self, slot: int) -> None:
        self.engine.close_slot(slot)

    def begin(self, slots, requests) -> None:
        self.sampler.begin(slots, [r.seed if r.seed is not None else fresh_seed() for r in requests])
        # the history of seen ids is only read by the repetition penalty
        self.track_seen = any(r.repetition_penalty != 1.0 for r in requests)

    def forward(self, slots, token_lists):
        logits = self.engine.step([StepEntry(s, t, [len(t) - 1]) for s, t in zip(slots, token_lists)])
        if self.track_seen:
            ctx = self.engine.last_context
            self.sampler.observe(ctx.tok_slot, ctx.token_ids)
        return logits

    def sample_begin(self, logits, slots, requests):
        """Launches the sampling of one id a sequence and the copy of the ids (with the device's error
        flag) to pinned host memory.  Nothing here waits for the device: the slots of the rows are the
        step's own device array, the options are cached on the device while they stay the same."""
        n = len(slots)
        device = self.engine.model.device
        if self._explicit_slots:
            row_slot = torch.tensor(slots, dtype=torch.int32, device=device)
            self._explicit_slots = False
        else:
            row_slot = self.engine.last_context.seq_slot[:n]
        ids = self.sampler.sample(logits[:n], row_slot, [r.sampler_config() for r in requests])
        if self._host is None or self._host.numel() < n + 1:
            self._host = torch.empty(max(64, n + 1), dtype=torch.int32, pin_memory=ids.is_cuda)
        self._host[:n].copy_(ids, non_blocking=True)
        self._host[n:n + 1].copy_(self.engine.model.error_flag, non_blocking=True)
        event = None
        if ids.is_cuda:
            event = torch.cuda.Event()
            event.record()
        return ids, n, event

    def sample_end(self, pending) -> list:
        """The ids of ``sample_begin`` on the host (one synchronisation, on the copy only)."""
        _, n, event = pending
        if event is not None:
            event.synchronize()
        out = self._host[:n].tolist()
        if int(self._host[n]) != 0:
            self.engine.check_errors()  # raises, and clears the flag
        return out

    def sample(self, logits, slots, requests) -> list:
        return self.sample_end(self.sample_begin(logits, slots, requests))

    def forward_sampled(self, slots, pending):
        """The next decode step of the same sequences, fed with the ids that ``sample_begin`` left
        on the device."""
        ids, n, _ = pending
        logits = self.engine.step_sampled(slots, ids[:n])
        if self.track_seen:
            ctx = self.engine.last_context
            self.sampler.observe(ctx.tok_slot, ctx.token_ids)
        return logits

    def rows(self, logits, rows):
        """Some rows of a step's logits (sequences that ended are dropped); the next sampling is told
        its slots explicitly."""
        self._explicit_slots = True
        return logits[torch.tensor(rows, dtype=torch.int64, device=logits.device)]


class Runtime:
    """A loaded model and the factory of sessions (crates/xrt-runtime/src/lib.rs:15-47)."""

    def __init__(self, model: Model, cache_tokens: int | None = None, max_batch: int = 64):
        self.model = model
        self.cache_tokens = cache_tokens
        self.max_batch = max_batch

    @classmethod
    def load(cls, path: str, dtype="bfloat16", device="cuda:0", cache_tokens: int | None = None,
             max_batch: int = 64) -> "Runtime":
        return cls(Model.load(path, dtype=dtype, device=device), cache_tokens, max_batch)

    def new_session(self) -> "Session":
        return Session(self)


class Session:
    """Generation for one request (``generate``, ``generate_stream``) or many (``generate_batch``)."""

    def __init__(self, runtime: Runtime):
        self.runtime = runtime
        self.backend: DeviceBackend | None = None
        self.last_stats = None

    def _backend_for(self, capacity: int) -> DeviceBackend:
        if self.backend is None or self.backend.engine.cache.capacity_tokens < capacity:
            self.backend = None  # let the old cache go before the new one is made
            self.backend = DeviceBackend(Engine(self.runtime.model, capacity, max_slots=self.runtime.max_batch))
        return self.backend

    def generate_batch(self, requests, on_token=None):
        """Returns (list of GenerateResult in request order, GenerateStats)."""
        model = self.runtime.model
        context = model.max_positions
        if not requests:
            raise RuntimeFault("no request to generate for")
        held = sorted((tokens_held(r, context) for r in requests), reverse=True)
        capacity = sum(held[: self.runtime.max_batch])
        if self.runtime.cache_tokens is not None:
            capacity = min(capacity, max(self.runtime.cache_tokens, held[0]))
        backend = self._backend_for(capacity)
        results, stats = generate(backend, requests, model.vocab_size, context, model.spec.stop_ids,
                                  capacity_tokens=backend.engine.cache.capacity_tokens,
                                  max_batch=self.runtime.max_batch, on_token=on_token)
        self.last_stats = stats
        return results, stats

    def generate_stream(self, request: GenerateRequest, on_token) -> None:
        """Calls ``on_token(token id)`` for each generated token (session.rs:69-197)."""
        self.generate_batch([request], on_token=lambda _, token: on_token(token))

    def generate(self, request: GenerateRequest) -> list:
        """The generated token ids of one request (session.rs:63-67)."""
        results, _ = self.generate_batch([request])
        return results[0].tokens
