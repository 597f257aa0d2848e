"""Choice among the bfloat16 matrix-product kernels.  ``run`` returns False when none of the
tensor-core kernels takes the shape, and the caller uses the CUDA-core kernel that takes any."""
from __future__ import annotations

from ..csrc import ops


def aligned(x, weight) -> bool:
    """16-byte rows for both operands: what the vector loads and TMA of the fast kernels need."""
    return (weight.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and weight.is_contiguous())


def run(out, x, weight, accumulate: bool) -> bool:
    if not aligned(x, weight):
        return False
    mode = "accumulate" if accumulate else "store"
    rows = x.shape[0]
    if rows <= ops.STREAM_MAX_ROWS:
        ops.gemm_stream(out, x, weight, mode)
        return True
    ops.gemm_tcgen05(out, x, weight, mode)
    return True


def run_swiglu(out, x, weight_gate_up, inner: int) -> bool:
    """out = silu(x . gate^T) * (x . up^T) for the fused weight [2 * inner, width]; False if no
    fused kernel takes the shape."""
    if not aligned(x, weight_gate_up):
        return False
    if x.shape[0] <= ops.STREAM_MAX_ROWS:
        ops.gemm_stream(out, x, weight_gate_up, "swiglu", up_rows=inner)
    else:
        ops.gemm_tcgen05(out, x, weight_gate_up, "swiglu", up_rows=inner)
    return True
