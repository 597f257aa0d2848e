"""Helpers for typed configurations read from a model folder's config.json."""
from __future__ import annotations

import json
import os
from typing import Any

from ..core import ConfigError

_MISSING = object()


class ModelConfig:
    """Base of every architecture's configuration class.

    A subclass is a frozen dataclass whose fields are the sizes and constants of
    the architecture, with ``from_dict`` reading the architecture's own
    config.json keys and ``to_dict`` writing them back.  Nothing outside the
    configuration may hold a size or constant that config.json gives.
    """

    architecture: str

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":  # pragma: no cover - interface
        raise NotImplementedError

    def to_dict(self) -> dict:  # pragma: no cover - interface
        raise NotImplementedError

    def with_stop_ids(self, ids: tuple) -> "ModelConfig":
        """The same configuration with ``ids`` as its stop ids (``eos_token_ids``)."""
        import dataclasses
        return dataclasses.replace(self, eos_token_ids=tuple(ids))


class KeyReader:
    """Reads keys of a config.json dict with type checks and collects what was wrong, so that one
    error can name every bad key at once."""

    def __init__(self, raw: dict, where: str = "config.json"):
        self.raw = raw
        self.where = where
        self.problems: list[str] = []

    def _get(self, key: str, default: Any):
        value = self.raw.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                self.problems.append(f"missing key {key!r}")
                return None
            return default
        return value

    def positive_int(self, key: str, default: Any = _MISSING):
        value = self._get(key, default)
        if value is None:
            return None
        if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
            self.problems.append(f"{key!r} must be a positive integer, got {value!r}")
            return None
        return value

    def number(self, key: str, default: Any = _MISSING, positive: bool = True):
        value = self._get(key, default)
        if value is None:
            return None
        if isinstance(value, bool) or not isinstance(value, (int, float)) or (positive and value <= 0):
            self.problems.append(f"{key!r} must be a positive number, got {value!r}")
            return None
        return float(value)

    def boolean(self, key: str, default: Any = _MISSING):
        value = self._get(key, default)
        if value is None:
            return None
        if not isinstance(value, bool):
            self.problems.append(f"{key!r} must be true or false, got {value!r}")
            return None
        return value

    def int_tuple(self, key: str) -> tuple:
        value = self.raw.get(key)
        if value is None:
            return ()
        if isinstance(value, int) and not isinstance(value, bool):
            return (value,)
        if isinstance(value, list) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
            return tuple(value)
        self.problems.append(f"{key!r} must be an integer or a list of integers, got {value!r}")
        return ()

    def fail(self, problem: str) -> None:
        self.problems.append(problem)

    def finish(self) -> None:
        if self.problems:
            raise ConfigError(f"{self.where}: " + "; ".join(self.problems))


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as fh:
            raw = json.load(fh)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return raw


def read_generation_stop_ids(folder: str) -> tuple:
    """``eos_token_id`` (an integer or a list) of the folder's generation_config.json; () if the
    file or the key is absent.  Folders of chat models keep the ids that end a turn there."""
    path = os.path.join(folder, "generation_config.json")
    if not os.path.exists(path):
        return ()
    try:
        with open(path) as fh:
            raw = json.load(fh)
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    reader = KeyReader(raw, where=path)
    ids = reader.int_tuple("eos_token_id")
    reader.finish()
    return ids
