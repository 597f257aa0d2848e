"""The sampler's options, with the names, defaults and meanings of the reference
(crates/xrt-runtime/src/sampler.rs:6-25)."""
from __future__ import annotations

from dataclasses import dataclass

from ..core import ConfigError

GREEDY_THRESHOLD = 1e-5  # temperature at or below this is greedy (sampler.rs:63)


@dataclass(frozen=True)
class SamplerConfig:
    """temperature 0.8 (<= 1e-5: argmax); top_k 40 (0: all); top_p 0.95 (>= 1: all);
    repetition_penalty 1.1 (<= 1: none; applies to every id of the prompt and of what was
    generated); seed None (a fresh one each request)."""
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    repetition_penalty: float = 1.1
    seed: int | None = None

    def validate(self) -> None:
        if self.temperature < 0 or self.temperature != self.temperature:
            raise ConfigError(f"temperature {self.temperature} must not be negative")
        if self.top_k < 0:
            raise ConfigError(f"top_k {self.top_k} must not be negative")
        if not (0 < self.top_p):
            raise ConfigError(f"top_p {self.top_p} must be positive")
        if self.repetition_penalty <= 0:
            raise ConfigError(f"repetition_penalty {self.repetition_penalty} must be positive")

    @property
    def greedy(self) -> bool:
        return self.temperature <= GREEDY_THRESHOLD
