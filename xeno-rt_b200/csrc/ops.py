"""Python bindings of the CUDA kernels: one function per exported launcher.

The kernels are plain ``extern "C"`` launchers that take device pointers, sizes and a stream; the
functions here check shapes, dtypes, contiguity and device of the torch tensors they are given,
pass the current torch stream and turn a refusal or launch error into ``KernelError``.  There is
no fallback: without a CUDA device or without the built library every function raises.
"""
from __future__ import annotations

import contextlib
import ctypes
import dataclasses
import threading

import torch

from ..core import KernelError
from . import build as _build

_lib = None
_lock = threading.Lock()
_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float

_CODES = {torch.float32: 0, torch.bfloat16: 1}

_SIGNATURES = {
    "xrt_embedding": [_P, _P, _P, _I, _I, _I, _I, _P, _P],
    "xrt_rmsnorm": [_P, _P, _P, _P, _I, _I, _F, _I, _I, _P],
    "xrt_swiglu": [_P, _P, _I, _I, _I, _I, _P],
    "xrt_rope_table": [_P, _P, _P, _F, _I, _I, _P],
    "xrt_qk_rope_kv_write": [_P, _P, _P, _P, _I, _I, _I, _P, _P, _F, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I,
                             _I, _I, _I, _I, _I, _P],
    "xrt_attention_reference": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _I, _P],
    "xrt_gemm_reference": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "xrt_gemm_stream": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "xrt_gemm_stream_norm": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _I, _P, _P],
    "xrt_gemm_stream_normed": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _I, _P, _P, _I, _F, _P],
    "xrt_gemm_tcgen05_normed": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _I, _P, _P, _I, _F, _P],
    "xrt_gemm_decode_tcgen05_normed": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _I, _F, _P],
    "xrt_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "xrt_gemm_decode_tcgen05": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "xrt_gemm_decode_tcgen05_norm": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _I, _P, _P],
    "xrt_gemm_decode_tcgen05_norm_parts": [_I, _I, _I, _I],
    "xrt_attention_decode_fused": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P, _I],
    "xrt_attention_decode": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P, _I],
    "xrt_attention_decode_qkv": [_P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _I, _F, _P, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I,
                                 _I, _I, _F, _I, _I, _I, _P, _P, _P, _I],
    "xrt_attention_prefill": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    "xrt_attention_prefill_tcgen05": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P],
    "xrt_fill_normal": [_P, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_double, ctypes.c_double, _I, _P],
    "xrt_sample": [_P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P],
    "xrt_mark_seen": [_P, _I, _P, _P, _I, _I, _P],
}


def library():
    """The loaded kernel library; builds it first if it is missing or stale."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.build()
            try:
                lib = ctypes.CDLL(path)
            except OSError as exc:
                raise KernelError(f"cannot load {path}: {exc}") from None
            for name, argtypes in _SIGNATURES.items():
                try:
                    fn = getattr(lib, name)
                except AttributeError:
                    raise KernelError(f"{path} does not export {name}") from None
                fn.argtypes = argtypes
                fn.restype = _I
            lib.xrt_attention_decode_fused_max_splits.argtypes = [_I, _I]
            lib.xrt_attention_decode_fused_max_splits.restype = _I
            lib.xrt_gemm_tcgen05_norm_parts.argtypes = [_I]
            lib.xrt_gemm_tcgen05_norm_parts.restype = _I
            lib.xrt_gemm_stream_norm_blocks.argtypes = [_I, _I]
            lib.xrt_gemm_stream_norm_blocks.restype = _I
            lib.xrt_set_tuning.argtypes = [_I, _I]
            lib.xrt_set_tuning.restype = _I
            lib.xrt_gemm_decode_tcgen05_scratch.argtypes = [_I, _I, _I, _I, _I]
            lib.xrt_gemm_decode_tcgen05_scratch.restype = ctypes.c_longlong
            lib.xrt_gemm_decode_tcgen05_plan.argtypes = [_I, _I, _I, _I, _I, ctypes.POINTER(ctypes.c_int)]
            lib.xrt_gemm_decode_tcgen05_plan.restype = _I
            _lib = lib
    return _lib


def _kernels():
    return library()


@dataclasses.dataclass(frozen=True)
class Tuning:
    """Which kernel variant runs where the library has several; the defaults are the measured
    choices.  Set with ``set_tuning`` (process-wide, since the parts call the kernels directly) or
    for a stretch of code with ``tuned(...)``; ``Engine(tuning=...)`` sets it when the engine is made.

    ``graphs``           decode steps are replayed from CUDA graphs
    ``pdl``              kernels of a step are launched with programmatic dependent launch
    ``decode_gemm``      "auto", or "stream" / "tcgen05" to force one of the few-row products
    ``decode_gemm_clusters``  splits of K of the tcgen05 few-row product meet through a cluster
    ``decode_attention`` "auto", "rows" (query heads as MMA rows), "cp" (cp.async tiles), "nocluster"
    ``prefill_attention`` "auto" or "mma" (the mma.sync kernel also where the tcgen05 one applies)
    ``gemm_tile_rows``   0 (auto), 128 or 256: the tile of the prompt product
    ``pending_norm``     "auto": a few-row product that adds into the residual prepares the norm that follows
                         it where the next product runs on the kernel that can finish it; "off": never
                         (a norm kernel runs); "force": wherever the kernels allow, whatever the sizes
    ``decode_cluster_pairs``  decode attention merges a (token, kv head)'s splits as one thread-block
                         cluster up to so many pairs a step; beyond, partials and a second kernel
    """
    graphs: bool = True
    pdl: bool = True
    decode_gemm: str = "auto"
    decode_gemm_clusters: bool = True
    decode_attention: str = "auto"
    prefill_attention: str = "auto"
    gemm_tile_rows: int = 0
    decode_cluster_pairs: int = 128
    pending_norm: str = "auto"


_DECODE_ATTENTION = {"auto": 0, "rows": 1, "cp": 2, "nocluster": 3}
_tuning = Tuning()


def tuning() -> Tuning:
    return _tuning


def set_tuning(new: Tuning) -> None:
    """Makes ``new`` the tuning of every later launch of this process."""
    global _tuning
    if new.decode_gemm not in ("auto", "stream", "tcgen05"):
        raise KernelError(f"tuning: decode_gemm {new.decode_gemm!r} is not auto, stream or tcgen05")
    if new.decode_attention not in _DECODE_ATTENTION:
        raise KernelError(f"tuning: decode_attention {new.decode_attention!r} is not one of {sorted(_DECODE_ATTENTION)}")
    if new.pending_norm not in ("auto", "off", "force"):
        raise KernelError(f"tuning: pending_norm {new.pending_norm!r} is not auto, off or force")
    if new.prefill_attention not in ("auto", "mma"):
        raise KernelError(f"tuning: prefill_attention {new.prefill_attention!r} is not auto or mma")
    lib = library()
    for key, value in ((0, int(new.pdl)), (1, _DECODE_ATTENTION[new.decode_attention]),
                       (2, int(new.gemm_tile_rows)), (3, int(new.decode_gemm_clusters)),
                       (4, int(new.decode_cluster_pairs))):
        if lib.xrt_set_tuning(key, value) != 0:
            raise KernelError(f"tuning: value {value} of setting {key} was refused")
    _tuning = new


@contextlib.contextmanager
def tuned(**changes):
    """``with tuned(prefill_attention="mma"): ...`` runs the body with these settings changed."""
    before = _tuning
    set_tuning(dataclasses.replace(before, **changes))
    try:
        yield
    finally:
        set_tuning(before)


def require_device() -> None:
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this library runs on the GPU only and has no CPU fallback")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _code(dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not handled by the kernels (float32, bfloat16)") from None


def _ptr(t, name: str, dtype=None) -> int:
    if t is None:
        return 0
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t.data_ptr()


_launches = 0


def launch_count() -> int:
    """How many kernels of this library were launched so far (a graph replay counts the kernels
    that were captured into it)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status == -1:
        raise KernelError(f"{what}: the kernel refused its arguments")
    if status == -2:
        raise KernelError(f"{what}: sizes or dtypes outside what the kernel handles")
    raise KernelError(f"{what}: CUDA launch error {status}")


def embedding(out, table, ids, error_flag) -> None:
    """out[t, :] = table[ids[t], :] as float32; raises error_flag[0] on an id outside the table."""
    n, hidden = out.shape
    vocab = table.shape[0]
    if table.shape[1] != hidden or ids.numel() != n:
        raise KernelError("embedding: shapes do not fit")
    _check(_kernels().xrt_embedding(_ptr(out, "out", torch.float32), _ptr(table, "table"),
                                   _ptr(ids, "ids", torch.int32), n, hidden, vocab, _code(table.dtype),
                                   _ptr(error_flag, "error_flag", torch.int32), _stream()), "embedding")


def rmsnorm(out, x, weight, eps: float, rows=None) -> None:
    """out[r] = rmsnorm(x[rows[r]] if rows is given else x[r]) * weight; x is float32."""
    n_rows, width = out.shape
    if x.shape[1] != width or weight.numel() != width or (rows is None and x.shape[0] != n_rows):
        raise KernelError("rmsnorm: shapes do not fit")
    if rows is not None and rows.numel() != n_rows:
        raise KernelError("rmsnorm: one row index per output row is needed")
    _check(_kernels().xrt_rmsnorm(_ptr(out, "out"), _ptr(x, "x", torch.float32), _ptr(weight, "weight"),
                                 _ptr(rows, "rows", torch.int32), n_rows, width, float(eps),
                                 _code(weight.dtype), _code(out.dtype), _stream()), "rmsnorm")


def swiglu(out, gate_up) -> None:
    """out[t, f] = silu(gate_up[t, f]) * gate_up[t, F + f]."""
    n, width = out.shape
    if gate_up.shape[0] != n or gate_up.shape[1] != 2 * width:
        raise KernelError("swiglu: shapes do not fit")
    _check(_kernels().xrt_swiglu(_ptr(out, "out"), _ptr(gate_up, "gate_up"), n, width, _code(gate_up.dtype),
                                _code(out.dtype), _stream()), "swiglu")


def rope_table(cos_sin, positions, freq, scale: float) -> None:
    """cos_sin[t, i] = (cos, sin)(positions[t] * scale / freq[i]); cos_sin is float32 [T, half, 2]."""
    n, half = cos_sin.shape[0], cos_sin.shape[1]
    if positions.numel() != n or freq.numel() != half or cos_sin.shape[2] != 2:
        raise KernelError("rope_table: shapes do not fit")
    _check(_kernels().xrt_rope_table(_ptr(cos_sin, "cos_sin", torch.float32),
                                    _ptr(positions, "positions", torch.int32), _ptr(freq, "freq", torch.float32),
                                    float(scale), n, half, _stream()), "rope_table")


def qk_rope_kv_write(q_out, k_pool, v_pool, qkv, k_offset: int, v_offset: int, q_norm_w, k_norm_w, eps: float,
                     cos_sin, tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int, head_dim: int,
                     write_kv: bool = True, pairing: str = "split_half") -> None:
    """Head norms, rotation, q output and cache write in one kernel; see rotary_kv.cu.  ``cos_sin``
    [T, rope_dim / 2, 2] rotates the first rope_dim dims of every head: pairs (i, i + rope_dim / 2)
    with ``pairing`` "split_half", pairs (2i, 2i + 1) with "interleaved"; the rest stays as it is."""
    if pairing not in ("split_half", "interleaved"):
        raise KernelError(f"qk_rope_kv_write: pairing {pairing!r} is not split_half or interleaved")
    n = qkv.shape[0]
    rope_half = 0 if cos_sin is None else cos_sin.shape[1]
    if q_out.shape != (n, n_heads * head_dim) or tok_slot.numel() != n or tok_pos.numel() != n:
        raise KernelError("qk_rope_kv_write: shapes do not fit")
    if write_kv:
        for pool in (k_pool, v_pool):
            if pool.dim() != 4 or pool.shape[1] != n_kv_heads or pool.shape[2] != 64 or pool.shape[3] != head_dim:
                raise KernelError("qk_rope_kv_write: the cache pool must be [blocks, kv heads, 64, head_dim]")
        if qkv.shape[1] < v_offset + n_kv_heads * head_dim:
            raise KernelError("qk_rope_kv_write: the q/k/v row is too short")
    norm_dtype = q_norm_w.dtype if q_norm_w is not None else torch.float32
    cache_dtype = k_pool.dtype if write_kv else q_out.dtype
    _check(_kernels().xrt_qk_rope_kv_write(
        _ptr(q_out, "q_out"), _ptr(k_pool if write_kv else None, "k_pool"),
        _ptr(v_pool if write_kv else None, "v_pool"), _ptr(qkv, "qkv", torch.float32), qkv.shape[1], k_offset,
        v_offset, _ptr(q_norm_w, "q_norm_w"), _ptr(k_norm_w, "k_norm_w"), float(eps),
        _ptr(cos_sin, "cos_sin", torch.float32), rope_half, _ptr(tok_slot, "tok_slot", torch.int32),
        _ptr(tok_pos, "tok_pos", torch.int32), _ptr(block_table, "block_table", torch.int32),
        block_table.shape[1], n, n_heads, n_kv_heads, head_dim, 1 if write_kv else 0,
        1 if pairing == "interleaved" else 0, _code(norm_dtype),
        _code(q_out.dtype), _code(cache_dtype), _stream()), "qk_rope_kv_write")


def attention_reference(out, q, k_pool, v_pool, tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int,
                        head_dim: int, scale: float, window: int = 0) -> None:
    """Causal GQA attention over the cache, one warp per (token, head); any dtype."""
    n = q.shape[0]
    if q.shape != (n, n_heads * head_dim) or out.shape != q.shape:
        raise KernelError("attention_reference: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_reference: the cache pool must be [blocks, kv heads, 64, head_dim]")
    _check(_kernels().xrt_attention_reference(
        _ptr(out, "out"), _ptr(q, "q"), _ptr(k_pool, "k_pool"), _ptr(v_pool, "v_pool", k_pool.dtype),
        _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n, n_heads, n_kv_heads, head_dim,
        float(scale), int(window), _code(q.dtype), _code(k_pool.dtype), _code(out.dtype), _stream()),
        "attention_reference")


def gemm_reference(out, x, w, accumulate: bool = False) -> None:
    """out = x . w^T (or out += x . w^T into a float32 out) with 32-bit fused multiply-adds."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: rows must be contiguous")
    if not x.is_cuda or not out.is_cuda:
        raise KernelError("gemm: operands must be on a CUDA device")
    _check(_kernels().xrt_gemm_reference(out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0),
                                        out.stride(0), _code(x.dtype), _code(w.dtype), _code(out.dtype),
                                        1 if accumulate else 0, _stream()), "gemm_reference")


STREAM_MAX_ROWS = 64
_error_flags: dict = {}


def error_flag(device) -> torch.Tensor:
    """The int32 flag of ``device`` that kernels raise when a bounded wait inside them ran out.
    Made when a model is built (never inside a stream capture)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def check_error_flag(device) -> None:
    """Reads the flag back (a synchronisation) and raises if a kernel raised it."""
    flag = error_flag(device)
    value = int(flag.item())
    if value != 0:
        flag.zero_()
        key = flag.device.index if flag.device.index is not None else torch.cuda.current_device()
        if key in _counters:  # a block that gave up never brought its tile's counter back to zero
            _counters[key].zero_()
        raise KernelError(f"a kernel reported error {value}: a bounded wait on a copy or a tensor-core operation ran "
                          f"out; results of the last steps are not valid")


DECODE_TCGEN05_MAX_ROWS = 128
_counters: dict = {}
_sm_counts: dict = {}
_COUNTER_SLOTS = 1 << 16


def device_state(device):
    """Per-device state of the kernels, made when a model is built (never inside a stream capture):
    the error flag, the tile counters of the split-K decode product (zero between launches) and
    the number of multiprocessors."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _counters:
        _counters[key] = torch.zeros(_COUNTER_SLOTS, dtype=torch.int32, device=device)
        _sm_counts[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return error_flag(device), _counters[key], _sm_counts[key]


_decode_plans: dict = {}


def gemm_decode_tcgen05_fill(sms: int, m: int, n: int, k: int, mode: str):
    """(rounds, share of the multiprocessor-rounds that do work) of ``gemm_decode_tcgen05`` on this
    product on a device of ``sms`` multiprocessors: its items (tiles of 128 weight rows x splits of
    K) run in rounds of one a multiprocessor.  Host arithmetic only: no device is needed."""
    return gemm_decode_tcgen05_plan(sms, m, n, k, mode)[:2]


def gemm_decode_tcgen05_plan(sms: int, m: int, n: int, k: int, mode: str):
    """(rounds, fill, kind of reduction) of ``gemm_decode_tcgen05`` on this product: the kind is "none" (K is not
    split), "cluster" (the splits of a tile meet as a thread-block cluster) or "scratch" (partial sums in
    global memory, merged by the block that brings a tile's last split)."""
    key = (sms, (m + 15) // 16, n, k, mode, tuning().decode_gemm_clusters)
    if key not in _decode_plans:
        plan = (ctypes.c_int * 3)()
        _check(library().xrt_gemm_decode_tcgen05_plan(m, n, k, {"store": 0, "accumulate": 1, "swiglu": 2}[mode], sms, plan),
               "gemm_decode_tcgen05_plan")
        items = plan[0] * plan[1]
        rounds = -(-items // sms)
        kind = "none" if plan[1] == 1 else ("cluster" if plan[2] else "scratch")
        _decode_plans[key] = (rounds, items / (rounds * sms), kind)
    return _decode_plans[key]


_decode_norm_parts: dict = {}


def gemm_decode_tcgen05_norm_parts(m: int, n: int, k: int, device) -> int:
    """How many partial sums of squares a row ``gemm_decode_tcgen05(..., norm=...)`` leaves, or 0 when
    that product cannot prepare a norm on this device (only splits of K that run as clusters do).
    Asks the device once for each class of sizes."""
    sms = device_state(device)[2]
    key = (sms, (m + 15) // 16, n, k, tuning().decode_gemm_clusters)
    if key not in _decode_norm_parts:
        with torch.cuda.device(device):
            _decode_norm_parts[key] = library().xrt_gemm_decode_tcgen05_norm_parts(int(m), int(n), int(k), sms)
    return _decode_norm_parts[key]


def gemm_decode_tcgen05(out, x, w, mode: str = "store", up_rows: int = 0, squares=None, eps: float = 0.0, norm=None) -> None:
    """bfloat16 product for at most 128 rows on the tcgen05 tensor cores with swapped operands:
    the weight is streamed once by TMA, K is split across blocks and summed in split order.
    ``squares`` (float32 [parts, rows], from a product with ``norm=...``): ``x`` is a residual times
    its norm weight, and every row's result is multiplied by 1 / sqrt(sum of its parts / K + eps).
    ``norm`` = (scaled, weight, squares) with "accumulate", where ``gemm_decode_tcgen05_norm_parts`` is
    not 0: the product prepares the RMSNorm that follows it, as ``gemm_stream`` does."""
    m, k = x.shape
    n = out.shape[1]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_decode_tcgen05: operands must be bfloat16")
    rows_needed = n + up_rows if mode == "swiglu" else n
    if w.shape[1] != k or w.shape[0] < rows_needed or out.shape[0] != m or (mode != "swiglu" and w.shape[0] != n):
        raise KernelError(f"gemm_decode_tcgen05: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1 or not x.is_cuda or not out.is_cuda:
        raise KernelError("gemm_decode_tcgen05: rows must be contiguous and on a CUDA device")
    if (n + 127) // 128 > _COUNTER_SLOTS:
        raise KernelError("gemm_decode_tcgen05: more tiles than counters")
    code = {"store": 0, "accumulate": 1, "swiglu": 2}[mode]
    flag, counters, sms = device_state(x.device)
    lib = library()
    floats = lib.xrt_gemm_decode_tcgen05_scratch(m, n, k, code, sms)
    partial = torch.empty(floats, dtype=torch.float32, device=x.device) if floats else None
    if squares is not None and (mode == "accumulate" or squares.dim() != 2 or squares.shape[1] != m):
        raise KernelError("gemm_decode_tcgen05: squares must be [parts, rows], and not with accumulate")
    if norm is not None:
        scaled, weight, emitted = norm
        parts = gemm_decode_tcgen05_norm_parts(m, n, k, x.device)
        if (mode != "accumulate" or out.dtype != torch.float32 or parts == 0 or scaled.shape != (m, n) or scaled.stride(1) != 1
                or weight.numel() != n or tuple(emitted.shape) != (parts, m) or not emitted.is_contiguous()):
            raise KernelError("gemm_decode_tcgen05: the buffers of the following norm do not fit the product")
        _check(lib.xrt_gemm_decode_tcgen05_norm(
            out.data_ptr(), x.data_ptr(), _ptr(w, "w"), _ptr(partial, "partial"), counters.data_ptr(), m, n, k, x.stride(0),
            out.stride(0), w.shape[0], sms, flag.data_ptr(), _ptr(scaled, "scaled", torch.bfloat16), scaled.stride(0),
            _ptr(weight, "weight"), _code(weight.dtype), _ptr(emitted, "squares", torch.float32), _stream()),
            "gemm_decode_tcgen05")
        return
    _check(lib.xrt_gemm_decode_tcgen05_normed(
        out.data_ptr(), x.data_ptr(), _ptr(w, "w"), _ptr(partial, "partial"), counters.data_ptr(), m, n, k, x.stride(0),
        out.stride(0), w.shape[0], _code(out.dtype), code, up_rows, sms, flag.data_ptr(),
        _ptr(squares, "squares", torch.float32), 0 if squares is None else squares.shape[0], float(eps), _stream()),
        "gemm_decode_tcgen05")


def gemm_tcgen05_norm_parts(n: int) -> int:
    """How many partial sums of squares a row ``gemm_tcgen05(..., norm=...)`` leaves (host arithmetic)."""
    return library().xrt_gemm_tcgen05_norm_parts(int(n))


def gemm_tcgen05(out, x, w, mode: str = "store", up_rows: int = 0, norm=None, squares=None, eps: float = 0.0) -> None:
    """bfloat16 product for many rows on the tcgen05 tensor cores with TMA-fed operands; modes as
    for ``gemm_stream``.  ``norm`` = (scaled, weight, squares) with "accumulate": the product prepares the
    RMSNorm that follows it (as ``gemm_stream`` does; ``squares`` is float32 [gemm_tcgen05_norm_parts(n), m]).
    ``squares`` (with "store" or "swiglu"): ``x`` is such a prepared input (as for ``gemm_decode_tcgen05``)."""
    m, k = x.shape
    n = out.shape[1]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tcgen05: operands must be bfloat16")
    rows_needed = n + up_rows if mode == "swiglu" else n
    if w.shape[1] != k or w.shape[0] < rows_needed or out.shape[0] != m or (mode != "swiglu" and w.shape[0] != n):
        raise KernelError(f"gemm_tcgen05: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1 or not x.is_cuda or not out.is_cuda:
        raise KernelError("gemm_tcgen05: rows must be contiguous and on a CUDA device")
    code = {"store": 0, "accumulate": 1, "swiglu": 2}[mode]
    flag = error_flag(x.device)
    scaled = weight = emitted = None
    if norm is not None:
        scaled, weight, emitted = norm
        if (mode != "accumulate" or scaled.shape != (m, n) or scaled.stride(1) != 1 or weight.numel() != n
                or tuple(emitted.shape) != (gemm_tcgen05_norm_parts(n), m)):
            raise KernelError("gemm_tcgen05: the buffers of the following norm do not fit the product")
    if squares is not None and (mode == "accumulate" or squares.dim() != 2 or squares.shape[1] != m):
        raise KernelError("gemm_tcgen05: squares must be [parts, rows], and not with accumulate")
    _check(_kernels().xrt_gemm_tcgen05_normed(
        out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0), out.stride(0), w.shape[0], _code(out.dtype), code,
        up_rows, flag.data_ptr(), _ptr(scaled, "scaled", torch.bfloat16), 0 if scaled is None else scaled.stride(0),
        _ptr(weight, "weight"), _code(weight.dtype) if weight is not None else 0, _ptr(emitted, "squares", torch.float32),
        _ptr(squares, "squares", torch.float32), 0 if squares is None else squares.shape[0], float(eps), _stream()),
        "gemm_tcgen05")


STREAM_NORM_MAX_ROWS = 16


def gemm_stream_norm_parts(m: int, n: int) -> int:
    """How many partial sums of squares a row ``gemm_stream(..., norm=...)`` leaves (host arithmetic)."""
    parts = library().xrt_gemm_stream_norm_blocks(int(m), int(n))
    if parts <= 0:
        raise KernelError("gemm_stream: a following norm can be prepared for at most 16 rows")
    return parts


def gemm_stream(out, x, w, mode: str = "store", up_rows: int = 0, norm=None, squares=None, eps: float = 0.0) -> None:
    """bfloat16 product for at most 64 rows that streams the weight once; ``mode`` is "store",
    "accumulate" (into a float32 out) or "swiglu" (out[m, n] = silu(x . w[n]) * (x . w[n + up_rows])).
    ``norm`` = (scaled, weight, squares) with "accumulate" and at most 16 rows: the product also
    prepares the RMSNorm that follows it: ``scaled`` (bfloat16 [m, n]) receives the new residual times
    ``weight`` ([n]), ``squares`` (float32 [gemm_stream_norm_parts(m, n), m]) its sums of squares.
    ``squares`` (float32 [parts, m], with "store" or "swiglu"): ``x`` is such a prepared input, and every
    row's result is multiplied by 1 / sqrt(sum of its parts / k + eps) (as for ``gemm_decode_tcgen05``)."""
    m, k = x.shape
    n = out.shape[1]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_stream: operands must be bfloat16")
    rows_needed = n + up_rows if mode == "swiglu" else n
    if w.shape[1] != k or w.shape[0] < rows_needed or out.shape[0] != m or (mode != "swiglu" and w.shape[0] != n):
        raise KernelError(f"gemm_stream: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1 or not x.is_cuda or not out.is_cuda:
        raise KernelError("gemm_stream: rows must be contiguous and on a CUDA device")
    code = {"store": 0, "accumulate": 1, "swiglu": 2}[mode]
    if squares is not None:
        if norm is not None or mode == "accumulate" or squares.dim() != 2 or squares.shape[1] != m or not squares.is_contiguous():
            raise KernelError("gemm_stream: squares must be [parts, rows], and not with accumulate or a following norm")
        _check(_kernels().xrt_gemm_stream_normed(
            out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0), out.stride(0), _code(out.dtype), code, up_rows,
            0, 0, 0, 0, 0, _ptr(squares, "squares", torch.float32), squares.shape[0], float(eps), _stream()), "gemm_stream")
        return
    if norm is None:
        _check(_kernels().xrt_gemm_stream(out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0), out.stride(0),
                                         _code(out.dtype), code, up_rows, _stream()), "gemm_stream")
        return
    scaled, weight, squares = norm
    if (mode != "accumulate" or scaled.shape != (m, n) or scaled.stride(1) != 1 or weight.numel() != n
            or tuple(squares.shape) != (gemm_stream_norm_parts(m, n), m)):
        raise KernelError("gemm_stream: the buffers of the following norm do not fit the product")
    _check(_kernels().xrt_gemm_stream_norm(
        out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0), out.stride(0), _code(out.dtype), code, up_rows,
        _ptr(scaled, "scaled", torch.bfloat16), scaled.stride(0), _ptr(weight, "weight"), _code(weight.dtype),
        _ptr(squares, "squares", torch.float32), _stream()), "gemm_stream")


def attention_decode(out, q, k_pool, v_pool, tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int,
                     head_dim: int, scale: float, window: int, chunk: int, n_splits: int, fused: bool = True,
                     clusters: bool = True) -> None:
    """bfloat16 attention of one token a sequence over its cache blocks, split along the keys.
    ``fused``: the splits are merged by the last block of each (token, kv head) instead of by a
    second kernel (needs the device's tile counters; falls back when there are too many).
    ``clusters`` False: the splits never merge as thread-block clusters (for sequences of very unequal
    lengths: a cluster holds its places until its longest block is done)."""
    n = q.shape[0]
    if q.shape != (n, n_heads * head_dim) or out.shape != q.shape or tok_slot.numel() != n or tok_pos.numel() != n:
        raise KernelError("attention_decode: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_decode: the cache pool must be [blocks, kv heads, 64, head_dim]")
    part_o = part_ml = None
    merged = ctypes.c_int(0)  # set by the launcher when the splits merged themselves as clusters
    flag = error_flag(q.device)
    if n_splits > 1:
        part_o = torch.empty(n * n_heads * n_splits * head_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n * n_heads * n_splits * 2, dtype=torch.float32, device=q.device)
    if fused and n_splits > 1 and n * n_kv_heads <= _COUNTER_SLOTS:
        _, counters, _ = device_state(q.device)
        _check(_kernels().xrt_attention_decode_fused(
            _ptr(out, "out", torch.bfloat16), _ptr(part_o, "part_o"), _ptr(part_ml, "part_ml"), counters.data_ptr(),
            _ptr(q, "q", torch.bfloat16), _ptr(k_pool, "k_pool", torch.bfloat16), _ptr(v_pool, "v_pool", torch.bfloat16),
            k_pool.shape[0], _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
            _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n, n_heads, n_kv_heads, head_dim,
            float(scale), int(window), int(chunk), int(n_splits), flag.data_ptr(), _stream(), ctypes.byref(merged),
            1 if clusters else 0), "attention_decode")
        if n_splits > 1 and not merged.value and n_splits > attention_decode_fused_max_splits(head_dim, n_heads // n_kv_heads):
            add_launches(1)  # too many splits for the merging block: the combine kernel ran
        return
    _check(_kernels().xrt_attention_decode(
        _ptr(out, "out", torch.bfloat16), _ptr(part_o, "part_o"), _ptr(part_ml, "part_ml"),
        _ptr(q, "q", torch.bfloat16), _ptr(k_pool, "k_pool", torch.bfloat16), _ptr(v_pool, "v_pool", torch.bfloat16),
        k_pool.shape[0], _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n, n_heads, n_kv_heads, head_dim,
        float(scale), int(window), int(chunk), int(n_splits), flag.data_ptr(), _stream(), ctypes.byref(merged),
        1 if clusters else 0), "attention_decode")
    if n_splits > 1 and not merged.value:
        add_launches(1)  # the combine kernel


def attention_decode_takes_qkv(n_heads: int, n_kv_heads: int, head_dim: int, rope_half: int, pairing: str) -> bool:
    """Whether ``attention_decode_qkv`` takes these sizes (the kernel fed by TMA does the step between
    the q/k/v product and attention itself): head size 64, 128 or 256, at most 8 query heads a kv head,
    a split-half rotation over the whole head or none, and no other decode attention kernel forced."""
    return (head_dim in (64, 128, 256) and n_heads // n_kv_heads <= 8 and rope_half in (0, head_dim // 2)
            and (pairing == "split_half" or rope_half == 0) and tuning().decode_attention in ("auto", "nocluster"))


def attention_decode_qkv(out, qkv, k_offset: int, v_offset: int, q_norm_w, k_norm_w, eps: float, cos_sin, k_pool, v_pool,
                         tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                         window: int, chunk: int, n_splits: int, write_kv: bool = True, fused: bool = True,
                         clusters: bool = True) -> None:
    """Decode attention straight from the 32-bit output of the q/k/v product: per-head norms, rotation,
    the newest key and value into the cache (unless ``write_kv`` is False) and attention over the cache
    in ONE kernel (csrc/attention_decode.cu).  ``qkv``: float32 [n, row] with q at 0, k at ``k_offset``,
    v at ``v_offset``.  Check ``attention_decode_takes_qkv`` first; other sizes raise."""
    n = qkv.shape[0]
    if out.shape != (n, n_heads * head_dim) or tok_slot.numel() != n or tok_pos.numel() != n:
        raise KernelError("attention_decode_qkv: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_decode_qkv: the cache pool must be [blocks, kv heads, 64, head_dim]")
    if ((write_kv and qkv.shape[1] < v_offset + n_kv_heads * head_dim) or qkv.shape[1] < n_heads * head_dim
            or (cos_sin is not None and cos_sin.shape[1] != head_dim // 2)):
        raise KernelError("attention_decode_qkv: the q/k/v row or the rotation table does not fit the heads")
    part_o = part_ml = None
    merged = ctypes.c_int(0)
    flag, counters, _ = device_state(qkv.device)
    if n_splits > 1:
        part_o = torch.empty(n * n_heads * n_splits * head_dim, dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty(n * n_heads * n_splits * 2, dtype=torch.float32, device=qkv.device)
    use_counters = fused and n_splits > 1 and n * n_kv_heads <= _COUNTER_SLOTS
    norm_dtype = q_norm_w.dtype if q_norm_w is not None else torch.float32
    _check(_kernels().xrt_attention_decode_qkv(
        _ptr(out, "out", torch.bfloat16), _ptr(part_o, "part_o"), _ptr(part_ml, "part_ml"),
        counters.data_ptr() if use_counters else 0, _ptr(qkv, "qkv", torch.float32), qkv.shape[1], int(k_offset),
        int(v_offset), _ptr(q_norm_w, "q_norm_w"), _ptr(k_norm_w, "k_norm_w", norm_dtype), _code(norm_dtype), float(eps),
        _ptr(cos_sin, "cos_sin", torch.float32), 1 if write_kv else 0, _ptr(k_pool, "k_pool", torch.bfloat16),
        _ptr(v_pool, "v_pool", torch.bfloat16), k_pool.shape[0], _ptr(tok_slot, "tok_slot", torch.int32),
        _ptr(tok_pos, "tok_pos", torch.int32), _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n,
        n_heads, n_kv_heads, head_dim, float(scale), int(window), int(chunk), int(n_splits), flag.data_ptr(), _stream(),
        ctypes.byref(merged), 1 if clusters else 0), "attention_decode_qkv")
    if n_splits > 1 and not merged.value and (
            not use_counters or n_splits > attention_decode_fused_max_splits(head_dim, n_heads // n_kv_heads)):
        add_launches(1)  # the combine kernel


def attention_decode_fused_max_splits(head_dim: int, group: int) -> int:
    """The most splits that the last block of a (token, kv head) can merge inside the attention
    kernel (its shared memory holds the splits' maxima and sums); host arithmetic only."""
    n = library().xrt_attention_decode_fused_max_splits(int(head_dim), int(group))
    if n < 0:
        raise KernelError("attention_decode_fused_max_splits: head size or group outside what the kernels take")
    return n


def attention_prefill(out, q, k_pool, v_pool, cu_seqlens, seq_slot, seq_start, block_table, max_new: int,
                      n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """bfloat16 causal attention of sequences laid end to end, each continuing at seq_start."""
    n = q.shape[0]
    n_seqs = seq_slot.numel()
    if q.shape != (n, n_heads * head_dim) or out.shape != q.shape or cu_seqlens.numel() != n_seqs + 1:
        raise KernelError("attention_prefill: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_prefill: the cache pool must be [blocks, kv heads, 64, head_dim]")
    _check(_kernels().xrt_attention_prefill(
        _ptr(out, "out", torch.bfloat16), _ptr(q, "q", torch.bfloat16), _ptr(k_pool, "k_pool", torch.bfloat16),
        _ptr(v_pool, "v_pool", torch.bfloat16), _ptr(cu_seqlens, "cu_seqlens", torch.int32),
        _ptr(seq_slot, "seq_slot", torch.int32), _ptr(seq_start, "seq_start", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n_seqs, int(max_new), n_heads,
        n_kv_heads, head_dim, float(scale), int(window), _stream()), "attention_prefill")


def attention_prefill_tcgen05(out, q, k_pool, v_pool, cu_seqlens, seq_slot, seq_start, block_table, max_new: int,
                              n_heads: int, n_kv_heads: int, head_dim: int, scale: float) -> None:
    """bfloat16 causal attention of sequences laid end to end on the tcgen05 tensor cores (head size 128)."""
    n = q.shape[0]
    n_seqs = seq_slot.numel()
    if q.shape != (n, n_heads * head_dim) or out.shape != q.shape or cu_seqlens.numel() != n_seqs + 1:
        raise KernelError("attention_prefill_tcgen05: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_prefill_tcgen05: the cache pool must be [blocks, kv heads, 64, head_dim]")
    flag = error_flag(q.device)
    _check(_kernels().xrt_attention_prefill_tcgen05(
        _ptr(out, "out", torch.bfloat16), _ptr(q, "q", torch.bfloat16), _ptr(k_pool, "k_pool", torch.bfloat16),
        _ptr(v_pool, "v_pool", torch.bfloat16), _ptr(cu_seqlens, "cu_seqlens", torch.int32),
        _ptr(seq_slot, "seq_slot", torch.int32), _ptr(seq_start, "seq_start", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], k_pool.shape[0], n, n_seqs, int(max_new),
        n_heads, n_kv_heads, head_dim, float(scale), flag.data_ptr(), _stream()), "attention_prefill_tcgen05")


def fill_normal(out, key: int, mean: float, std: float) -> None:
    """Fills ``out`` with the seeded normal stream ``key`` (see weights/random_init.py)."""
    _check(_kernels().xrt_fill_normal(_ptr(out, "out"), out.numel(), key & ((1 << 64) - 1), float(mean),
                                     float(std), _code(out.dtype), _stream()), "fill_normal")


def sample(out_ids, logits, row_slot, temperature, top_k, top_p, penalty, seen, rng_key, rng_counter) -> None:
    """One token id per row of float32 logits; see sampling.cu for the conventions."""
    n, vocab = logits.shape
    seen_words = 0 if seen is None else seen.shape[1]
    _check(_kernels().xrt_sample(
        _ptr(out_ids, "out_ids", torch.int32), _ptr(logits, "logits", torch.float32), n, vocab,
        _ptr(row_slot, "row_slot", torch.int32), _ptr(temperature, "temperature", torch.float32),
        _ptr(top_k, "top_k", torch.int32), _ptr(top_p, "top_p", torch.float32),
        _ptr(penalty, "penalty", torch.float32), _ptr(seen, "seen", torch.int32), seen_words,
        _ptr(rng_key, "rng_key", torch.int64), _ptr(rng_counter, "rng_counter", torch.int32), _stream()), "sample")


def mark_seen(seen, slots, ids, vocab: int) -> None:
    """Sets the bit of ids[i] in the bitmap of slots[i]."""
    n = ids.numel()
    _check(_kernels().xrt_mark_seen(_ptr(seen, "seen", torch.int32), seen.shape[1],
                                   _ptr(slots, "slots", torch.int32), _ptr(ids, "ids", torch.int32), n, vocab,
                                   _stream()), "mark_seen")
