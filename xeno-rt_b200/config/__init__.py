"""Typed configurations and the one registry from an architecture's name to its model."""
from .base import ModelConfig, read_config_json
from .registry import (Architecture, register_architecture, get_architecture, architecture_names,
                       config_from_dict, load_config)

__all__ = ["ModelConfig", "read_config_json", "Architecture", "register_architecture",
           "get_architecture", "architecture_names", "config_from_dict", "load_config"]
