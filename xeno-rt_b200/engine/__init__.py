"""The model instance, the step function and the generation loop."""
from .model import Model
from .step import Engine, StepEntry, build_context

__all__ = ["Model", "Engine", "StepEntry", "build_context"]
