"""Arrangements: how the parts of one layer are put together around the residual stream."""
from __future__ import annotations

from dataclasses import dataclass

from .registry import register_part


@dataclass
class LayerParts:
    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object


def prenorm_residual(parts: LayerParts, x, ctx, store, owns_cache: bool) -> None:
    """x += mixer(norm(x)); x += feed_forward(norm(x))   (crates/xrt-models/src/llama.rs:433-602).
    ``x`` is the float32 residual stream and is updated in place; the sums are 32-bit."""
    parts.mixer.forward(parts.mixer_norm.forward(x), x, ctx, store, owns_cache)
    parts.ffn.forward(parts.ffn_norm.forward(x), x, ctx)


register_part("arrangement", "prenorm_residual", prenorm_residual)
