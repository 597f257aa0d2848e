"""Choice among the bfloat16 matrix-product kernels.  ``run`` returns False when none of the
tensor-core kernels takes the shape, and the caller uses the CUDA-core kernel that takes any.

Up to 128 rows (decode steps): the weight-streaming tcgen05 kernel with swapped operands and split
K (the batch is the MMA's N, so its time stays the time to read the weight); its splits of a tile
meet through a thread-block cluster's shared memory.  The products that add into the residual
stream are the exception up to 16 rows: there the cp.async weight-streaming kernel is faster
(measured over whole steps of 1 to 16 sequences at the 8B shape: the others gain 1 to 11 % on the
tcgen05 kernel, these lose 2 to 5 %).  More rows (prompts): the tiled tcgen05 kernel.
``XRT_DECODE_GEMM=stream`` or ``tcgen05`` forces one of the two decode kernels wherever it applies,
for comparison."""
from __future__ import annotations

import os

from ..csrc import ops

FORCE = os.environ.get("XRT_DECODE_GEMM", "")
STREAM_ROWS = 16  # products that add into the residual stream stay on the cp.async kernel up to here


def aligned(x, weight) -> bool:
    """16-byte rows for both operands: what the vector loads and TMA of the fast kernels need."""
    return (weight.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and weight.is_contiguous())


def _product(out, x, weight, mode: str, up_rows: int = 0) -> None:
    rows = x.shape[0]
    if FORCE == "stream":
        stream_rows = ops.STREAM_MAX_ROWS
    elif FORCE == "tcgen05":
        stream_rows = 0
    else:
        stream_rows = STREAM_ROWS if mode == "accumulate" else 0
    if rows <= stream_rows:
        ops.gemm_stream(out, x, weight, mode, up_rows)
    elif rows <= ops.DECODE_TCGEN05_MAX_ROWS:
        ops.gemm_decode_tcgen05(out, x, weight, mode, up_rows)
    else:
        ops.gemm_tcgen05(out, x, weight, mode, up_rows)


def run(out, x, weight, accumulate: bool) -> bool:
    if not aligned(x, weight):
        return False
    _product(out, x, weight, "accumulate" if accumulate else "store")
    return True


def run_swiglu(out, x, weight_gate_up, inner: int) -> bool:
    """out = silu(x . gate^T) * (x . up^T) for the fused weight [2 * inner, width]; False if no
    fused kernel takes the shape."""
    if not aligned(x, weight_gate_up):
        return False
    _product(out, x, weight_gate_up, "swiglu", inner)
    return True
