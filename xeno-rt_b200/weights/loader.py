"""Binding the tensors of a model folder to the tensors a model expects, by name.

A folder holds either one ``model.safetensors`` or an index ``model.safetensors.index.json`` whose
``weight_map`` sends each tensor name to one of several shard files.  The reference's contract is
"a path goes in, a model comes out" (crates/xrt-runtime/src/lib.rs:21-30): it maps the file, looks each
name up in a map and fails on the first missing one (crates/xrt-gguf/src/lib.rs:248-476, 532-541)
without checking shapes at load (crates/xrt-models/src/llama.rs:297-378, debug asserts at 1059-1060).
Here the headers of all files are checked at once and ONE error lists every missing tensor, every
unexpected tensor, every wrong shape and every disagreement between the index and its shards.

Tensors go to the device one at a time through a small staging buffer (pinned when the device is a
GPU), so the host never holds more than that buffer beside the memory maps.  Tensors that a part
wants side by side in one matrix (q, k and v; gate and up) are copied straight into their rows of
one device buffer: no second copy exists at any time.
"""
from __future__ import annotations

import fnmatch
import json
import os
from dataclasses import dataclass

import torch

from ..core import DType, WeightError, log
from .safetensors_io import TensorFile, read_safetensors_header, stored_dtype

MODEL_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"
STAGING_BYTES = 32 << 20  # one staging buffer; two are in use
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


def tensor_problems(expected: list[ExpectedTensor], header: dict, ignorable=()) -> list[str]:
    """The lines of the error: missing, unexpected, wrong shape or dtype; empty if all fits."""
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
    lines = []
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
    return lines


def check_tensors(expected: list[ExpectedTensor], header: dict, ignorable=(), where: str = "model file") -> None:
    """Raises one WeightError that lists all that does not fit; returns None if all fits."""
    lines = tensor_problems(expected, header, ignorable)
    if lines:
        raise WeightError("\n".join([f"{where} does not fit the model:"] + lines))


def kept_dtype(kind: str, stored: torch.dtype, compute: DType) -> torch.dtype:
    """The dtype a tensor is kept in on the device (see ExpectedTensor)."""
    if kind == "int":
        return torch.int32
    if compute is DType.F32:
        return torch.float32
    if kind == "vector" and stored == torch.float32:
        return torch.float32
    return torch.bfloat16


def locate_tensors(folder: str) -> tuple[dict, dict, list[str], str]:
    """Reads the headers of the folder's model file(s).  Returns (header, file of each tensor,
    problem lines, what to call the source in messages).  ``header`` is the union of the shards'
    headers; the problems are the disagreements between an index and its shards: a shard file that
    does not exist, a tensor that the index sends to a shard that does not hold it, a tensor that
    two shards hold, a tensor of a shard that the index does not list."""
    index_path = os.path.join(folder, INDEX_FILE)
    single = os.path.join(folder, MODEL_FILE)
    if not os.path.exists(index_path):
        header, _ = read_safetensors_header(single)
        return header, {name: single for name in header}, [], single
    try:
        with open(index_path) as fh:
            index = json.load(fh)
    except json.JSONDecodeError as exc:
        raise WeightError(f"{index_path}: not valid JSON ({exc})") from None
    weight_map = index.get("weight_map") if isinstance(index, dict) else None
    if not isinstance(weight_map, dict) or not all(isinstance(v, str) for v in weight_map.values()):
        raise WeightError(f"{index_path}: 'weight_map' must map tensor names to shard file names")
    problems: list[str] = []
    header: dict = {}
    where: dict = {}
    shard_headers: dict = {}
    for shard in sorted(set(weight_map.values())):
        path = os.path.join(folder, shard)
        if os.path.basename(shard) != shard:
            problems.append(f"  shard name {shard!r} is not a plain file name")
        elif not os.path.exists(path):
            problems.append(f"  missing shard file: {shard}")
        else:
            shard_headers[shard] = read_safetensors_header(path)[0]
    twice, unlisted = [], []
    for shard, shard_header in shard_headers.items():
        for name, meta in shard_header.items():
            if name in header:
                twice.append(f"{name} ({os.path.basename(where[name])} and {shard})")
                continue
            if name not in weight_map:
                unlisted.append(f"{name} ({shard})")
            header[name] = meta
            where[name] = os.path.join(folder, shard)
    absent = sorted(f"{name} ({shard})" for name, shard in weight_map.items()
                    if shard in shard_headers and name not in shard_headers[shard])
    for name, shard in weight_map.items():  # what the index says wins where a tensor is held twice
        if shard in shard_headers and name in shard_headers[shard]:
            header[name], where[name] = shard_headers[shard][name], os.path.join(folder, shard)
    if absent:
        problems.append(f"  listed in the index but absent from their shard ({len(absent)}): " + ", ".join(absent))
    if twice:
        problems.append(f"  held by two shards ({len(twice)}): " + ", ".join(sorted(twice)))
    if unlisted:
        problems.append(f"  held by a shard but not listed in the index ({len(unlisted)}): " + ", ".join(sorted(unlisted)))
    return header, where, problems, index_path


class LoadedTensors(dict):
    """{tensor name: device tensor}; ``fused`` maps a tuple of tensor names to the one buffer that
    holds them row block after row block (each name's tensor is then a view of its rows)."""

    def __init__(self):
        super().__init__()
        self.fused: dict[tuple, torch.Tensor] = {}


class _Stager:
    """Copies bytes of a memory map into a device tensor in pieces of at most STAGING_BYTES through
    two staging buffers used in turn (pinned for a GPU, so the copies run while the next piece is
    read from the file).  ``peak`` is the most staging memory that was ever in use."""

    def __init__(self, device, piece: int | None = None):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.piece = piece or STAGING_BYTES
        self.buffers = [None, None]
        self.events = [None, None]
        self.turn = 0
        self.peak = 0

    def _buffer(self, i: int, n: int) -> torch.Tensor:
        if self.events[i] is not None:
            self.events[i].synchronize()
            self.events[i] = None
        if self.buffers[i] is None or self.buffers[i].numel() < n:
            self.buffers[i] = torch.empty(n, dtype=torch.uint8, pin_memory=self.cuda)
            self.peak = max(self.peak, sum(b.numel() for b in self.buffers if b is not None))
        return self.buffers[i][:n]

    def copy(self, dest_bytes: torch.Tensor, source: TensorFile, name: str) -> None:
        """dest_bytes: a contiguous uint8 view of the destination, as long as the tensor's data."""
        total = source.nbytes(name)
        if dest_bytes.numel() != total:
            raise WeightError(f"{name}: {total} bytes in the file, {dest_bytes.numel()} expected")
        for begin in range(0, total, self.piece):
            n = min(self.piece, total - begin)
            view = source.bytes_of(name, begin, n)
            if not self.cuda:
                dest_bytes[begin:begin + n] = torch.from_numpy(view.copy())
                self.peak = max(self.peak, n)
                continue
            i, self.turn = self.turn, 1 - self.turn
            buf = self._buffer(i, n)
            buf.numpy()[:] = view
            dest_bytes[begin:begin + n].copy_(buf, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
            self.events[i] = event

    def finish(self) -> None:
        for event in self.events:
            if event is not None:
                event.synchronize()
        self.events = [None, None]


def load_weights(folder: str, expected: list[ExpectedTensor], compute: DType, device, ignorable=(),
                 fused_groups=(), stats: dict | None = None) -> LoadedTensors:
    """Reads the model file(s) of ``folder``, checks them against ``expected`` and returns
    {name: device tensor} in the kept dtypes.  ``fused_groups``: tuples of tensor names that are
    to lie one after another (along their rows) in one buffer.  ``stats`` (a dict) receives
    ``peak_staging_bytes``: the most host memory the copies held at once."""
    header, where, problems, source = locate_tensors(folder)
    problems += tensor_problems(expected, header, ignorable)
    if problems:
        raise WeightError("\n".join([f"{source} does not fit the model:"] + problems))
    by_name = {e.name: e for e in expected}
    skipped = [n for n in header if n not in by_name]
    if skipped:
        log("debug", f"ignored tensors: {', '.join(sorted(skipped))}")

    out = LoadedTensors()
    device = torch.device(device)

    def kept(e: ExpectedTensor) -> torch.dtype:
        return kept_dtype(e.kind, stored_dtype(header[e.name]["dtype"]), compute)

    for group in fused_groups:
        members = [by_name[n] for n in group]
        dtypes = {kept(e) for e in members}
        tails = {tuple(e.shape[1:]) for e in members}
        if len(dtypes) != 1 or len(tails) != 1 or any(len(e.shape) < 1 for e in members):
            raise WeightError(f"tensors {list(group)} cannot share one buffer: their row shapes or dtypes differ")
        if any(n in out for n in group):
            raise WeightError(f"tensors {list(group)}: a tensor is asked into two shared buffers")
        rows = sum(e.shape[0] for e in members)
        buffer = torch.empty((rows,) + next(iter(tails)), dtype=next(iter(dtypes)), device=device)
        begin = 0
        for e in members:
            out[e.name] = buffer[begin:begin + e.shape[0]]
            begin += e.shape[0]
        out.fused[tuple(group)] = buffer
    stager = _Stager(device)
    files: dict[str, TensorFile] = {}
    try:
        # file by file, in the order of the data inside each file: sequential reads
        order = sorted(expected, key=lambda e: (where[e.name], header[e.name]["data_offsets"][0]))
        for e in order:
            path = where[e.name]
            if path not in files:
                files[path] = TensorFile(path)
            stored = stored_dtype(header[e.name]["dtype"])
            dest = out.get(e.name)
            if dest is None:
                dest = out[e.name] = torch.empty(e.shape, dtype=kept(e), device=device)
            if dest.dtype == stored:
                stager.copy(dest.reshape(-1).view(torch.uint8), files[path], e.name)
            else:  # the stored form visits the device, is converted there and dropped
                raw = torch.empty(e.shape, dtype=stored, device=device)
                stager.copy(raw.reshape(-1).view(torch.uint8), files[path], e.name)
                dest.copy_(raw)
                del raw
        stager.finish()
    finally:
        for f in files.values():
            f.close()
    if stats is not None:
        stats["peak_staging_bytes"] = stager.peak
        stats["files"] = len(files)
    return out
