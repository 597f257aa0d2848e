"""The registry from an architecture's name (``architectures[0]`` of config.json) to its model.

The reference decides with an ``if`` over two names (crates/xrt-models/src/llama.rs:43-51) and
answers ``Unsupported`` for anything else; here a table does, so that another architecture is one
``register_architecture`` call in a module of its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from ..core import ConfigError, Unsupported
from .base import ModelConfig, read_config_json, read_generation_stop_ids


@dataclass(frozen=True)
class Architecture:
    """One entry: the config class that reads config.json and the function that turns a config
    into a ``ModelSpec`` (the layer-by-layer description that the engine builds parts from)."""
    name: str
    config_class: type
    build_spec: Callable


_REGISTRY: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable) -> Architecture:
    if name in _REGISTRY:
        raise ConfigError(f"architecture {name!r} is registered already")
    entry = Architecture(name, config_class, build_spec)
    _REGISTRY[name] = entry
    return entry


def architecture_names() -> list[str]:
    return sorted(_REGISTRY)


def get_architecture(name: str) -> Architecture:
    try:
        return _REGISTRY[name]
    except KeyError:
        raise Unsupported(f"architecture {name!r} is not supported; supported: "
                          f"{', '.join(architecture_names())}") from None


def config_from_dict(raw: dict) -> tuple[Architecture, ModelConfig]:
    names = raw.get("architectures")
    if not isinstance(names, list) or not names or not isinstance(names[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    arch = get_architecture(names[0])
    return arch, arch.config_class.from_dict(raw)


def load_config(folder: str) -> tuple[Architecture, ModelConfig]:
    """The folder's config.json as a typed configuration.  Its stop ids are config.json's
    ``eos_token_id`` followed by those of generation_config.json that it does not name already
    (the reference takes its one id from the model file, crates/xrt-runtime/src/session.rs:110)."""
    arch, config = config_from_dict(read_config_json(folder))
    extra = read_generation_stop_ids(folder)
    if extra:
        own = tuple(getattr(config, "eos_token_ids", ()))
        config = config.with_stop_ids(own + tuple(i for i in extra if i not in own))
    return arch, config
