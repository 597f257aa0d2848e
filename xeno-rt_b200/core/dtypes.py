"""The two compute dtypes of the library and their names in files and on the command line."""
from __future__ import annotations

import enum

from .errors import ConfigError


class DType(enum.Enum):
    """Compute dtype of a model instance.  ``code`` is the integer the CUDA kernels take."""
    F32 = ("float32", 0)
    BF16 = ("bfloat16", 1)

    @property
    def label(self) -> str:
        return self.value[0]

    @property
    def code(self) -> int:
        return self.value[1]


_ALIASES = {"float32": DType.F32, "fp32": DType.F32, "f32": DType.F32,
            "bfloat16": DType.BF16, "bf16": DType.BF16}


def parse_dtype(name) -> DType:
    if isinstance(name, DType):
        return name
    try:
        return _ALIASES[str(name).lower().replace("torch.", "")]
    except KeyError:
        raise ConfigError(f"dtype {name!r} is not one of {sorted(_ALIASES)}") from None


def torch_dtype(dtype: DType):
    import torch
    return torch.float32 if dtype is DType.F32 else torch.bfloat16


def safetensors_code(dtype: DType) -> str:
    return "F32" if dtype is DType.F32 else "BF16"
