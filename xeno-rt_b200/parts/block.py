"""Arrangements: how the parts of one layer are put together around the residual stream."""
from __future__ import annotations

from .registry import register_part


class LayerParts:
    """The built parts of one layer by the names its ``LayerSpec`` gave them: ``parts.mixer`` or
    ``parts["mixer"]``; ``parts.names()`` in the spec's order; ``parts.role(name)``."""

    def __init__(self, parts: dict, roles: dict | None = None):
        self._parts = dict(parts)
        self._roles = dict(roles or {})

    def __getattr__(self, name):
        try:
            return self.__dict__["_parts"][name]
        except KeyError:
            raise AttributeError(f"the layer has no part named {name!r}; it has {list(self.__dict__['_parts'])}") from None

    def __getitem__(self, name):
        return self._parts[name]

    def __contains__(self, name) -> bool:
        return name in self._parts

    def names(self) -> list:
        return list(self._parts)

    def role(self, name: str) -> str:
        return self._roles.get(name, "")

    def values(self):
        return self._parts.values()


def prenorm_residual(parts: LayerParts, x, ctx, stores, owns_cache: bool) -> None:
    """x += mixer(norm(x)); x += feed_forward(norm(x))   (crates/xrt-models/src/llama.rs:433-602).
    ``x`` is the float32 residual stream and is updated in place; the sums are 32-bit.  ``stores``
    maps a part's name to the cache storage it asked for."""
    h = ctx.take_pending(parts.mixer_norm)  # the layer before may have prepared this layer's first norm
    if h is None:
        h = parts.mixer_norm.forward(x)
    ctx.then_norm = _norm_that_can_wait(parts.ffn_norm, parts.ffn, ctx, x)
    parts.mixer.forward(h, x, ctx, stores.get("mixer"), owns_cache)
    h = ctx.take_pending(parts.ffn_norm)
    if h is None:
        h = parts.ffn_norm.forward(x)
    after = ctx.shared.get("next_layer")  # (norm, the part that takes its result) of the layer that runs next
    ctx.then_norm = _norm_that_can_wait(after[0], after[1], ctx, x) if after else None
    parts.ffn.forward(h, x, ctx)


def _norm_that_can_wait(norm, consumer, ctx, x):
    """``norm`` if the part that adds into the residual before it may prepare it (so that no norm
    kernel runs in between): the part that takes the norm's result must say that it can finish it."""
    can = getattr(consumer, "takes_pending_norm", None)
    return norm if can is not None and can(ctx.n_tokens, x.device) else None


# what a layer of this arrangement begins with: the norm it applies to the residual stream first, and the
# part that takes that norm's result
prenorm_residual.first_norm = lambda parts: (parts.mixer_norm, parts.mixer)
register_part("arrangement", "prenorm_residual", prenorm_residual)
