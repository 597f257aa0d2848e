"""Registries of part kinds, one for each role.  A part class is registered under a name; a
``PartSpec`` picks it by that name.  Tests register toy parts here without touching the package.

Roles and the interface each class must have (all take ``(params, weights, dtype, device)`` in
``__init__``, where ``weights`` maps the part's tensor roles to device tensors, and all have a
``weight_shapes(params)`` class method returning ``{tensor role: (shape, kind)}`` with kind one of
"matrix", "vector", "int"):

norm            ``forward(x, rows=None) -> normed``: x is the float32 residual stream [T, D];
                the result has the compute dtype; ``rows`` (int32 device tensor) gathers rows.
mixer           ``cache_need() -> KVNeed | StateNeed | list of them | None`` and
                ``forward(h, residual, ctx, store, owns_cache) -> None``: adds its result into the
                float32 ``residual`` [T, D] in place; ``store`` is the cache storage it asked for
                (a list of storages if it asked with a list).
feed_forward    ``forward(h, residual, ctx) -> None``: adds its result into ``residual``.
position        ``tables(ctx) -> tensor | None``: per-step rotation table [T, half, 2] of
                (cos, sin), cached in ``ctx.shared``; None means no rotation.
embedding       ``forward(token_ids, error_flag) -> x`` float32 [T, D].
lm_head         ``forward(normed) -> logits`` float32 [R, V].
A part class may set ``graph_safe = True`` to say that its ``forward`` only launches device work
in stream order whose shapes depend on nothing but the number of tokens and the context bucket (no
reads back to the host, no data-dependent Python branches); decode steps of a model whose parts
all say so are captured in CUDA graphs, any other model runs every step kernel by kernel.

arrangement     a function ``(layer_parts, x, ctx, stores, owns_cache) -> None`` that runs one layer:
                ``layer_parts`` holds every part of the layer by the name its LayerSpec gave it,
                ``stores`` maps a part's name to the cache storage that part asked for.
A part class may have ``fused_weights(params) -> {role: (roles, ...)}``: tensors that it wants one after
another (along rows) in one buffer; when the loader could arrange that, ``weights[role]`` is that buffer.
"""
from __future__ import annotations

from ..core import ConfigError

ROLES = ("norm", "mixer", "feed_forward", "position", "embedding", "lm_head", "arrangement")
_REGISTRY: dict[str, dict[str, object]] = {role: {} for role in ROLES}


def register_part(role: str, kind: str, cls, replace: bool = False):
    if role not in _REGISTRY:
        raise ConfigError(f"unknown part role {role!r}; roles: {ROLES}")
    if kind in _REGISTRY[role] and not replace:
        raise ConfigError(f"{role} part {kind!r} is registered already")
    _REGISTRY[role][kind] = cls
    return cls


def part_class(role: str, kind: str):
    try:
        return _REGISTRY[role][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(role, {}))) or "none"
        raise ConfigError(f"no {role} part named {kind!r}; registered: {known}") from None


def part_kinds(role: str) -> list[str]:
    return sorted(_REGISTRY[role])
