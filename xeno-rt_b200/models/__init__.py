"""Architectures: each module holds a configuration class and the function that turns it into a
``ModelSpec``, and registers both under the architecture's name."""
from . import llama  # registers LlamaForCausalLM and Qwen3ForCausalLM

__all__ = ["llama"]
