"""Seeded random weights: a model folder (config.json + model.safetensors) from a configuration
and a seed, and the generator behind it.

The reference has random weights in a test fixture only, from a linear congruential generator
(tests/common/mod.rs:719-731).  This library's generator is counter-based, so that any element
of any tensor can be drawn alone, on the host or by a CUDA kernel, with the same result:

    key(name)   = splitmix64(seed XOR fnv1a64(name))
    bits(i)     = splitmix64(key + (i + 1) * 0x9E3779B97F4A7C15)          (all modulo 2^64)
    u1          = ((bits >> 32) + 1) / 2^32        in (0, 1]
    u2          = (bits & 0xFFFFFFFF) / 2^32       in [0, 1)
    z(i)        = sqrt(-2 ln u1) * cos(2 pi u2)    in float64 (Box-Muller, one draw an element)
    value(i)    = mean + std * z(i), rounded to float32 and then to the stored dtype

Matrices and the embedding are N(0, 0.02); norm weights are 1 + N(0, 0.1).
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch

from ..core import DType, torch_dtype

INIT_MATRIX_STD = 0.02
INIT_NORM_STD = 0.1
_GOLDEN = 0x9E3779B97F4A7C15
_MASK = (1 << 64) - 1


def _splitmix64_int(x: int) -> int:
    x = (x + _GOLDEN) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def _fnv1a64(text: str) -> int:
    h = 0xCBF29CE484222325
    for byte in text.encode():
        h = ((h ^ byte) * 0x100000001B3) & _MASK
    return h


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of one tensor's stream."""
    return _splitmix64_int((seed & _MASK) ^ _fnv1a64(name))


def _splitmix64_np(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = x + np.uint64(_GOLDEN)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def normal_values(key: int, count: int, mean: float, std: float, start: int = 0) -> np.ndarray:
    """Elements start .. start+count of the stream ``key`` as float32."""
    with np.errstate(over="ignore"):
        idx = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        bits = _splitmix64_np(np.uint64(key) + idx * np.uint64(_GOLDEN))
    u1 = ((bits >> np.uint64(32)).astype(np.float64) + 1.0) / 4294967296.0
    u2 = (bits & np.uint64(0xFFFFFFFF)).astype(np.float64) / 4294967296.0
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (mean + std * z).astype(np.float32)


def random_tensors(expected, seed: int, dtype: DType) -> dict[str, torch.Tensor]:
    """CPU tensors for every expected tensor: vectors 1 + N(0, 0.1), all else N(0, 0.02)."""
    out = {}
    for e in expected:
        count = int(np.prod(e.shape, dtype=np.int64))
        if e.kind == "vector":
            values = normal_values(tensor_key(seed, e.name), count, 1.0, INIT_NORM_STD)
        else:
            values = normal_values(tensor_key(seed, e.name), count, 0.0, INIT_MATRIX_STD)
        out[e.name] = torch.from_numpy(values).reshape(e.shape).to(torch_dtype(dtype))
    return out


def write_random_model(folder: str, config, seed: int, dtype=DType.F32, shards: int = 1) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration or
    a config.json dict) with weights drawn from ``seed``; returns the folder.  With ``shards`` > 1
    the tensors go into that many shard files beside an index, as large checkpoints are stored."""
    from ..config import config_from_dict
    from ..core import parse_dtype, safetensors_code
    from .safetensors_io import write_safetensors, write_sharded_safetensors

    dtype = parse_dtype(dtype)
    raw = config if isinstance(config, dict) else config.to_dict()
    arch, typed = config_from_dict(raw)
    spec = arch.build_spec(typed)
    os.makedirs(folder, exist_ok=True)
    out_config = typed.to_dict()
    out_config["torch_dtype"] = dtype.label
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(out_config, fh, indent=2)
    tensors = random_tensors(spec.expected_tensors(), seed, dtype)
    metadata = {"format": "pt", "seed": seed, "dtype": safetensors_code(dtype)}
    if shards > 1:
        write_sharded_safetensors(folder, tensors, shards, metadata)
    else:
        write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata)
    return folder
