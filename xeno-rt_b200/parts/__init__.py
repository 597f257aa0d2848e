"""Parts that layers are put together from: norms, position encodings, mixers, feed-forwards,
embedding and output head, and arrangements; their specs and registries."""
from .spec import PartSpec, LayerSpec, SchedulePlace, ModelSpec, prenorm_layer
from .registry import register_part, part_class, part_kinds, ROLES
from .context import StepContext
from .linear import linear
from . import norm, rotary, embedding, attention, feed_forward, block  # registers the built-in parts
from .block import LayerParts

__all__ = ["PartSpec", "LayerSpec", "prenorm_layer", "SchedulePlace", "ModelSpec", "register_part", "part_class", "part_kinds",
           "ROLES", "StepContext", "linear", "LayerParts"]
