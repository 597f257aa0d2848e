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
    parts.mixer.forward(parts.mixer_norm.forward(x), x, ctx, stores.get("mixer"), owns_cache)
    parts.ffn.forward(parts.ffn_norm.forward(x), x, ctx)


register_part("arrangement", "prenorm_residual", prenorm_residual)
