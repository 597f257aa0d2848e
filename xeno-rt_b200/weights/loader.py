"""Binding the tensors of a model file to the tensors a model expects, by name.

The reference looks each name up in a map and fails on the first missing one
(crates/xrt-gguf/src/lib.rs:532-541) without checking shapes at load
(crates/xrt-models/src/llama.rs:297-378, debug asserts at 1059-1060).  Here the whole file is
checked at once and ONE error lists every missing tensor, every unexpected tensor and every
wrong shape.
"""
from __future__ import annotations

import fnmatch
import os
from dataclasses import dataclass

import torch

from ..core import DType, WeightError, log
from .safetensors_io import read_safetensors, read_safetensors_header

MODEL_FILE = "model.safetensors"
_FLOAT_CODES = ("F32", "BF16", "F16")
_INT_CODES = ("I32", "I64")


@dataclass(frozen=True)
class ExpectedTensor:
    """What a part asks of the file for one of its tensors.

    ``kind`` decides the dtype it is kept in: a ``matrix`` (operand of a matrix product) is kept
    in the compute dtype; a ``vector`` (norm weights and the like) stored in 32-bit stays 32-bit
    and is otherwise kept in the compute dtype; an ``int`` table is kept as int32.
    """
    name: str
    shape: tuple
    kind: str = "matrix"


def check_tensors(expected: list[ExpectedTensor], header: dict, ignorable=(), where: str = "model file") -> None:
    """Raises one WeightError that lists all that does not fit; returns None if all fits."""
    wanted = {e.name: e for e in expected}
    missing = sorted(n for n in wanted if n not in header)
    unexpected = sorted(n for n in header if n not in wanted
                        and not any(fnmatch.fnmatchcase(n, pat) for pat in ignorable))
    wrong = []
    for name, e in sorted(wanted.items()):
        meta = header.get(name)
        if meta is None:
            continue
        if tuple(meta["shape"]) != tuple(e.shape):
            wrong.append(f"{name}: shape {list(meta['shape'])}, expected {list(e.shape)}")
        elif e.kind == "int" and meta["dtype"] not in _INT_CODES:
            wrong.append(f"{name}: dtype {meta['dtype']}, expected an integer table")
        elif e.kind != "int" and meta["dtype"] not in _FLOAT_CODES:
            wrong.append(f"{name}: dtype {meta['dtype']}, expected one of {list(_FLOAT_CODES)}")
    if not (missing or unexpected or wrong):
        return
    parts = [f"{where} does not fit the model:"]
    if missing:
        parts.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        parts.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        parts.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
    raise WeightError("\n".join(parts))


def kept_dtype(kind: str, stored: torch.dtype, compute: DType) -> torch.dtype:
    """The dtype a tensor is kept in on the device (see ExpectedTensor)."""
    if kind == "int":
        return torch.int32
    if compute is DType.F32:
        return torch.float32
    if kind == "vector" and stored == torch.float32:
        return torch.float32
    return torch.bfloat16


def load_weights(folder: str, expected: list[ExpectedTensor], compute: DType, device, ignorable=()) -> dict:
    """Reads ``model.safetensors`` of ``folder``, checks it against ``expected`` and returns
    {name: device tensor} in the kept dtypes."""
    path = os.path.join(folder, MODEL_FILE)
    header, _ = read_safetensors_header(path)
    check_tensors(expected, header, ignorable, where=path)
    names = {e.name for e in expected}
    skipped = [n for n in header if n not in names]
    if skipped:
        log("debug", f"ignored tensors: {', '.join(sorted(skipped))}")
    host = read_safetensors(path, names)
    out = {}
    for e in expected:
        t = host[e.name]
        out[e.name] = t.to(device=device, dtype=kept_dtype(e.kind, t.dtype, compute)).contiguous()
    return out
