"""Choice among the bfloat16 matrix-product kernels.  ``run`` returns False when none of the
tensor-core kernels takes the shape, and the caller uses the CUDA-core kernel that takes any.

17 to 128 rows (decode steps of many sequences): the weight-streaming tcgen05 kernel with swapped
operands and split K (the batch is the MMA's N, so its time stays the time to read the weight); its
splits of a tile meet through a thread-block cluster's shared memory.  Up to 16 rows that kernel or
the cp.async weight-streaming kernel, whichever suits the product (``tcgen05_for_few_rows``).  More
than 128 rows (prompts): the tiled tcgen05 kernel.  ``ops.Tuning.decode_gemm`` = "stream" or "tcgen05"
forces one of the two decode kernels wherever it applies, for comparison."""
from __future__ import annotations

from ..csrc import ops

STREAM_ROWS = 16  # up to here the cp.async kernel is a candidate


def aligned(x, weight) -> bool:
    """16-byte rows for both operands: what the vector loads and TMA of the fast kernels need."""
    return (weight.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and weight.is_contiguous())


ACCUMULATE_MIN_K = 16384


def tcgen05_for_few_rows(sms: int, rows: int, n: int, k: int, mode: str) -> bool:
    """Up to 16 rows both decode kernels take the product.  The tcgen05 kernel runs its items one a
    multiprocessor in rounds: it wins where they fill the rounds (one round at least 0.6 full, or
    several at least 0.85 full).  Products that add into the residual stream stay on the cp.async
    kernel unless K is long (it slows down with K: 2.6 TB/s at K = 25,600, where the tcgen05 kernel
    reaches 4 TB/s).  Whole steps of 8 sequences at a width of 5,120 and an inner size of 25,600 went
    from 18.0 to 15.8 ms with this rule, and at 4,096 / 14,336 from 4.62 to 4.40 ms; with the limit at
    8,192 instead the first gains another 1.5 % and single sequences at the second lose 4.5 %."""
    if mode == "accumulate" and k < ACCUMULATE_MIN_K:
        return False
    rounds, fill = ops.gemm_decode_tcgen05_fill(sms, rows, n, k, mode)
    return fill >= 0.6 and (rounds == 1 or fill >= 0.85)


def _product(out, x, weight, mode: str, up_rows: int = 0) -> None:
    rows = x.shape[0]
    force = ops.tuning().decode_gemm
    if force == "stream":
        stream_rows = ops.STREAM_MAX_ROWS
    elif force == "tcgen05":
        stream_rows = 0
    elif rows > STREAM_ROWS:
        stream_rows = 0
    else:
        sms = ops.device_state(x.device)[2]
        stream_rows = 0 if tcgen05_for_few_rows(sms, rows, out.shape[1], x.shape[1], mode) else STREAM_ROWS
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
