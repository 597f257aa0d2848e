"""Minimal safetensors / config.json reader of the plain implementation.

Independent of the product's loader on purpose: a fault in the product's file
handling cannot hide behind a shared reader.  Format: 8-byte little-endian
header length, a JSON header {name: {dtype, shape, data_offsets}}, raw
little-endian data.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_model_folder(folder: str):
    """Returns (config dict, {tensor name: float32 ndarray})."""
    with open(os.path.join(folder, "config.json")) as fh:
        config = json.load(fh)
    path = os.path.join(folder, "model.safetensors")
    with open(path, "rb") as fh:
        (header_len,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(header_len))
        data = fh.read()
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = data[lo:hi]
        if meta["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(np.float32)
        elif meta["dtype"] == "BF16":
            arr = _bf16_to_f32(np.frombuffer(buf, dtype="<u2"))
        elif meta["dtype"] == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(np.float32)
        else:
            raise ValueError(f"plain reader: dtype {meta['dtype']} of {name}")
        tensors[name] = arr.reshape(meta["shape"])
    return config, tensors
