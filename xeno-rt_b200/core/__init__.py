"""Core types shared by every other part: errors, dtype names, logging.

Plays the role of the reference's ``xrt-core`` crate (crates/xrt-core/src/lib.rs):
``DType`` (lib.rs:10-110), ``XrtError`` (lib.rs:203-227).
"""
from .errors import (XrtError, ConfigError, WeightError, CacheError, KernelError, RuntimeFault,
                     Unsupported)
from .dtypes import DType, parse_dtype, torch_dtype, safetensors_code
from .log import log, log_level

__all__ = ["XrtError", "ConfigError", "WeightError", "CacheError", "KernelError", "RuntimeFault",
           "Unsupported", "DType", "parse_dtype", "torch_dtype", "safetensors_code", "log", "log_level"]
