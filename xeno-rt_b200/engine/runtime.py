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

    def open_slot(self) -> int:
        return self.engine.open_slot()

    def close_slot(self, slot: int) -> None:
        self.engine.close_slot(slot)

    def begin(self, slots, requests) -> None:
        self.sampler.begin(slots, [r.seed if r.seed is not None else fresh_seed() for r in requests])

    def forward(self, slots, token_lists):
        logits = self.engine.step([StepEntry(s, t, [len(t) - 1]) for s, t in zip(slots, token_lists)])
        ctx = self.engine.last_context
        self.sampler.observe(ctx.tok_slot, ctx.token_ids)
        return logits

    def sample(self, logits, slots, requests) -> list:
        n = len(slots)
        row_slot = torch.tensor(slots, dtype=torch.int32, device=self.engine.model.device)
        ids = self.sampler.sample(logits[:n], row_slot, [r.sampler_config() for r in requests])
        out = ids.tolist()
        self.engine.check_errors()
        return out


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
        if self.backend is None or self.backend.engine.cache.n_blocks * 64 < capacity:
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
                                  capacity_tokens=backend.engine.cache.n_blocks * 64,
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
