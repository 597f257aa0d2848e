"""xeno-rt_b200: a small model library with generation of its own for one B200.

It covers everything between a request's tokens and its next token for the Llama / Qwen3 dense
decoder of the reference (crates/xrt-models/src/llama.rs): a typed configuration and an
architecture registry (``config``), weights from safetensors (``weights``), layers assembled from
parts (``parts``), a block cache with one slot a sequence (``cache``), one step function and a
generation loop (``engine``), sampling (``sampling``) and hand-written CUDA kernels for sm_100a
(``csrc``).  The folder is imported as ``xeno_rt_b200``.
"""
from .core import (XrtError, ConfigError, WeightError, CacheError, KernelError, RuntimeFault, Unsupported,
                   DType, parse_dtype)

__version__ = "0.1.0"
from . import models  # registers the architectures
from .config import load_config, config_from_dict, register_architecture
from .engine import (Model, Engine, StepEntry, Runtime, Session, GenerateRequest, GenerateResult)
from .sampling import SamplerConfig
from .weights import write_random_model
