"""The model instance, the step function, the generation loop and the Python entry point."""
from .model import Model
from .step import Engine, StepEntry, build_context
from .generate import (GenerateRequest, GenerateResult, GenerateStats, SequenceProgress, generate,
                       plan_batches, tokens_held, validate_request)
from .runtime import Runtime, Session, DeviceBackend

__all__ = ["Model", "Engine", "StepEntry", "build_context", "GenerateRequest", "GenerateResult", "GenerateStats",
           "SequenceProgress", "generate", "plan_batches", "tokens_held", "validate_request", "Runtime", "Session",
           "DeviceBackend"]
