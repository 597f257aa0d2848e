"""The description of a model as data: which parts each layer is made of, with which sizes and
constants and which tensors, and the order in which layers run.

An architecture module turns its configuration into a ``ModelSpec``; the engine builds the parts
that the spec names from the registries of ``parts.registry``.  No part knows which model it is in.

The reference has one fixed block (crates/xrt-models/src/llama.rs:433-602) and one ``if`` for the
optional q/k norm (488-496); here every layer has its own ``LayerSpec``, so layers of one model may
differ in mixer, feed-forward or sizes, and the order of execution is a list that may name a
layer twice or let a place read the cache that another place owns.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..weights.loader import ExpectedTensor


@dataclass
class PartSpec:
    """One part: ``kind`` is its name in the registry of its role, ``params`` its sizes and
    constants, ``weights`` maps the part's tensor roles to tensor names in the model file."""
    kind: str
    params: dict = field(default_factory=dict)
    weights: dict = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One layer: its parts by name, ``{name: (role, PartSpec)}`` in the order they are built, and
    the ``arrangement`` that runs them around the residual stream.  The arrangement receives all of
    the layer's parts, so a layer with more norms, two mixers side by side or no feed-forward is
    another arrangement over another dict and nothing else."""
    parts: dict
    arrangement: str = "prenorm_residual"


def prenorm_layer(mixer_norm: PartSpec, mixer: PartSpec, ffn_norm: PartSpec, ffn: PartSpec) -> LayerSpec:
    """The layer of crates/xrt-models/src/llama.rs:433-602: a mixer and a feed-forward, each behind
    a norm, each added to the residual stream."""
    return LayerSpec({"mixer_norm": ("norm", mixer_norm), "mixer": ("mixer", mixer),
                      "ffn_norm": ("norm", ffn_norm), "ffn": ("feed_forward", ffn)}, "prenorm_residual")


@dataclass
class SchedulePlace:
    """One place in the order of execution: run ``layer``; ``cache_from`` = None means the place
    owns cache storage of its own, a number means it reads (and does not write) the storage that
    the earlier place of that index owns."""
    layer: int
    cache_from: int | None = None


@dataclass
class ModelSpec:
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: list
    schedule: list
    final_norm: PartSpec
    lm_head: PartSpec
    stop_ids: tuple = ()
    ignorable_tensors: tuple = ()

    def part_specs(self):
        """Every (role, spec) of the model, each weight-bearing part once."""
        yield "embedding", self.embedding
        for layer in self.layers:
            for role, part in layer.parts.values():
                yield role, part
        yield "norm", self.final_norm
        yield "lm_head", self.lm_head

    def expected_tensors(self) -> list[ExpectedTensor]:
        """What the model file must hold; a tensor named by two parts (a tied output matrix) is
        listed once and must have the same shape for both."""
        from .registry import part_class
        from ..core import ConfigError

        seen: dict[str, ExpectedTensor] = {}
        for role, spec in self.part_specs():
            cls = part_class(role, spec.kind)
            for tensor_role, (shape, kind) in cls.weight_shapes(spec.params).items():
                name = spec.weights.get(tensor_role)
                if name is None:
                    raise ConfigError(f"{role} part {spec.kind!r}: no tensor name for its {tensor_role!r}")
                e = ExpectedTensor(name, tuple(shape), kind)
                if name in seen and seen[name] != e:
                    raise ConfigError(f"tensor {name} is used with two shapes: {seen[name].shape} and {e.shape}")
                seen[name] = e
        return list(seen.values())

    def fused_groups(self) -> list[tuple]:
        """Tuples of tensor names that a part wants one after another in one buffer (its class says
        so with ``fused_weights``); the loader then reads them straight into that buffer."""
        from .registry import part_class

        groups = []
        for role, spec in self.part_specs():
            fused = getattr(part_class(role, spec.kind), "fused_weights", None)
            for roles in (fused(spec.params).values() if fused else ()):
                names = tuple(spec.weights[r] for r in roles)
                if names not in groups:
                    groups.append(names)
        return groups

    def validate(self) -> None:
        from ..core import ConfigError
        for i, place in enumerate(self.schedule):
            if not (0 <= place.layer < len(self.layers)):
                raise ConfigError(f"schedule place {i} names layer {place.layer}, the model has {len(self.layers)}")
            if place.cache_from is not None:
                if not (0 <= place.cache_from < i):
                    raise ConfigError(f"schedule place {i} reads the cache of place {place.cache_from}, "
                                      f"which does not come before it")
                if self.schedule[place.cache_from].cache_from is not None:
                    raise ConfigError(f"schedule place {i} reads the cache of place {place.cache_from}, "
                                      f"which owns none")
