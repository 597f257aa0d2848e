"""Arrangements: how the parts of one layer are put together around the residual stream."""
from __future__ import annotations

from ..csrc import ops
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
    mask = ops.tuning().prefetch if ctx.n_tokens <= 64 else 0
    if mask & 1:
        ops.hint_prefetch(getattr(parts.mixer, "first_weight", None), 0, 48 << 20)
    h = parts.mixer_norm.forward(x)
    parts.mixer.forward(h, x, ctx, stores.get("mixer"), owns_cache)
    if mask & 2:
        ops.hint_prefetch(getattr(parts.ffn, "first_weight", None), 0, 32 << 20)
    h = parts.ffn_norm.forward(x)
    parts.ffn.forward(h, x, ctx)


register_part("arrangement", "prenorm_residual", prenorm_residual)
