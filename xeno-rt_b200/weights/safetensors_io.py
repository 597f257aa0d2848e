"""The safetensors container, read and written directly.

Layout: an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` (plus an optional
``__metadata__`` entry), then the raw little-endian tensor bytes.  The reference reads
GGUF only (crates/xrt-gguf/src/lib.rs:248-476); safetensors is this library's input format.
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np
import torch

from ..core import WeightError

_ITEMSIZE = {"F32": 4, "BF16": 2, "F16": 2, "I32": 4, "I64": 8}
_TORCH = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32,
          "I64": torch.int64}
_CODE = {v: k for k, v in _TORCH.items()}


def read_safetensors_header(path: str) -> tuple[dict, int]:
    """Returns ({name: {"dtype", "shape", "data_offsets"}}, offset of the data section)."""
    try:
        size = os.path.getsize(path)
        with open(path, "rb") as fh:
            prefix = fh.read(8)
            if len(prefix) < 8:
                raise WeightError(f"{path}: shorter than a safetensors header")
            (header_len,) = struct.unpack("<Q", prefix)
            if header_len > size - 8:
                raise WeightError(f"{path}: header length {header_len} exceeds the file size {size}")
            header = json.loads(fh.read(header_len))
    except FileNotFoundError:
        raise WeightError(f"{path}: no such file") from None
    except json.JSONDecodeError as exc:
        raise WeightError(f"{path}: the header is not valid JSON ({exc})") from None
    header.pop("__metadata__", None)
    data_start = 8 + header_len
    for name, meta in header.items():
        code = meta.get("dtype")
        if code not in _ITEMSIZE:
            raise WeightError(f"{path}: tensor {name} has dtype {code}, supported: {sorted(_ITEMSIZE)}")
        lo, hi = meta["data_offsets"]
        count = int(np.prod(meta["shape"], dtype=np.int64)) if meta["shape"] else 1
        if hi - lo != count * _ITEMSIZE[code] or data_start + hi > size or lo < 0:
            raise WeightError(f"{path}: tensor {name} has data offsets {lo}..{hi} that do not fit its "
                              f"shape {meta['shape']} and dtype {code}, or the file")
    return header, data_start


class TensorFile:
    """One safetensors file kept open as a read-only memory map, so that a tensor's bytes are
    paged in only when they are asked for and no more of the file is ever held than the caller
    copies out."""

    def __init__(self, path: str):
        self.path = path
        self.header, self.data_start = read_safetensors_header(path)
        self._fh = open(path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)

    def nbytes(self, name: str) -> int:
        lo, hi = self.header[name]["data_offsets"]
        return hi - lo

    def bytes_of(self, name: str, begin: int = 0, count: int | None = None) -> np.ndarray:
        """A uint8 view (no copy) of ``count`` bytes of tensor ``name`` from byte ``begin`` on."""
        lo, hi = self.header[name]["data_offsets"]
        count = hi - lo - begin if count is None else count
        if begin < 0 or count < 0 or begin + count > hi - lo:
            raise WeightError(f"{self.path}: bytes {begin}..{begin + count} are outside tensor {name}")
        return np.frombuffer(self._map, dtype=np.uint8, count=count, offset=self.data_start + lo + begin)

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:  # a view handed out is still alive; the map goes with it
                pass
            self._map = None
            self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def stored_dtype(code: str) -> torch.dtype:
    return _TORCH[code]


def read_safetensors(path: str, names=None) -> dict[str, torch.Tensor]:
    """Reads tensors (all, or those in ``names``) as CPU torch tensors of their stored dtype."""
    header, data_start = read_safetensors_header(path)
    out: dict[str, torch.Tensor] = {}
    with open(path, "rb") as fh:
        mapped = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            for name, meta in header.items():
                if names is not None and name not in names:
                    continue
                lo, hi = meta["data_offsets"]
                raw = np.frombuffer(mapped, dtype=np.uint8, count=hi - lo, offset=data_start + lo).copy()
                tensor = torch.from_numpy(raw).view(_TORCH[meta["dtype"]]).reshape(meta["shape"])
                out[name] = tensor
        finally:
            mapped.close()
    return out


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Writes CPU tensors in name order; data begins on an 8-byte boundary."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _CODE:
            raise WeightError(f"cannot write tensor {name} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _CODE[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            fh.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def write_sharded_safetensors(folder: str, tensors: dict[str, torch.Tensor], n_shards: int,
                              metadata: dict | None = None) -> list[str]:
    """Writes ``tensors`` as ``model-0000i-of-0000n.safetensors`` files with about equal bytes each
    (in name order) and the index ``model.safetensors.index.json`` whose ``weight_map`` sends each
    name to its file.  Returns the shard file names."""
    import json as _json
    names = sorted(tensors)
    n_shards = max(1, min(int(n_shards), len(names)))
    total = sum(tensors[n].numel() * tensors[n].element_size() for n in names)
    shards: list[dict] = [{} for _ in range(n_shards)]
    used, k = 0, 0
    for i, name in enumerate(names):
        left_names, left_shards = len(names) - i, n_shards - k
        if shards[k] and k + 1 < n_shards and (used >= total * (k + 1) / n_shards or left_names < left_shards):
            k += 1
        shards[k][name] = tensors[name]
        used += tensors[name].numel() * tensors[name].element_size()
    files = [f"model-{i + 1:05d}-of-{n_shards:05d}.safetensors" for i in range(n_shards)]
    weight_map = {}
    for file, part in zip(files, shards):
        write_safetensors(os.path.join(folder, file), part, metadata)
        weight_map.update({name: file for name in part})
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as fh:
        _json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, fh, indent=1, sort_keys=True)
    return files
