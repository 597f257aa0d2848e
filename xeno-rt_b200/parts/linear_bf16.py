"""Choice among the bfloat16 matrix-product kernels.  ``run`` returns False when none of the
tensor-core kernels takes the shape, and the caller uses the CUDA-core kernel that takes any.

17 to 128 rows (decode steps of many sequences): the weight-streaming tcgen05 kernel with swapped
operands and split K (the batch is the MMA's N, so its time stays the time to read the weight); its
splits of a tile meet through a thread-block cluster's shared memory.  Up to 16 rows that kernel or
the cp.async weight-streaming kernel, whichever suits the product (``tcgen05_for_few_rows``).  More
than 128 rows (prompts): the tiled tcgen05 kernel.  ``ops.Tuning.decode_gemm`` = "stream" or "tcgen05"
forces one of the two decode kernels wherever it applies, for comparison."""
from __future__ import annotations

import torch

from ..csrc import ops

STREAM_ROWS = 16  # up to here the cp.async kernel is a candidate


def aligned(x, weight) -> bool:
    """16-byte rows for both operands: what the vector loads and TMA of the fast kernels need."""
    return (weight.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and weight.is_contiguous())


ACCUMULATE_MIN_K_9_ROWS = 8192  # a product of 9 to 16 rows that adds into the residual stream takes the tcgen05 kernel from here on
STREAM_BLOCKS_PER_SM = 4        # blocks of the cp.async kernel that a multiprocessor holds at once (registers)


def stream_kernel_waves(sms: int, n: int, accumulate: bool = False) -> float:
    """How full the cp.async kernel's rounds of blocks are for ``n`` weight rows (8 rows a block): 1 when all
    blocks run at once, else rounds / whole rounds.  640 blocks on 592 places are two rounds, the second
    nearly empty: such a product runs at half its rate (measured: 84 MB in 33 microseconds).  A product
    that adds into the residual stream takes 16 rows a block where that makes one round of it (three
    such blocks a multiprocessor), as ``csrc/gemm_stream.cu:stream_row_groups_accumulate`` decides."""
    blocks = -(-n // 8)
    if accumulate and blocks > sms * STREAM_BLOCKS_PER_SM and -(-n // 16) <= sms * 3:
        return 1.0
    waves = blocks / (sms * STREAM_BLOCKS_PER_SM)
    return 1.0 if waves <= 1.0 else waves / -(-waves // 1)


def tcgen05_for_few_rows(sms: int, rows: int, n: int, k: int, mode: str) -> bool:
    """Up to 16 rows both decode kernels take the product.  The tcgen05 kernel runs its items one a
    multiprocessor in rounds: it wins where they fill the rounds (one round at least 0.6 full, or
    several at least 0.85 full).  Products that add into the residual stream stay on the cp.async
    kernel up to 8 rows, and from 9 rows on below K = 8,192 (its time grows with the rows, the tcgen05
    kernel's does not), unless its own rounds of blocks are badly filled.  Measured alone and back to
    back, cp.async against tcgen05 in microseconds at 1 / 8 / 16 rows: N 4,096, K 4,096: 7.6 / 8.6 / 10.3
    against 11.5; K 14,336: 22.7 / 26.1 / 29.2 against 26.4; N 5,120, K 8,192: 15.0 / 16.6 / 21.4 against
    21.2; K 25,600: 44.7 / 48.4 / 66.7 against 55.0."""
    rounds, fill, reduction = ops.gemm_decode_tcgen05_plan(sms, rows, n, k, mode)
    fills = fill >= 0.6 and (rounds == 1 or fill >= 0.85)
    if mode == "accumulate" and (rows <= 8 or k < ACCUMULATE_MIN_K_9_ROWS):
        return fills and fill > stream_kernel_waves(sms, n, accumulate=True) + 0.2
    if mode == "store" and reduction == "scratch":
        # splits that the device does not hold as clusters end in one block that merges a tile: the cp.async
        # kernel with 16 weight rows a block is faster then (N 6,144, K 4,096, alone at 1 / 8 / 16 rows: 8.4 /
        # 8.9 / 9.7 against 14.4 us; whole steps of 1 / 8 / 16 sequences 3.27 -> 3.12, 3.90 -> 3.78, 4.77 -> 4.69
        # ms, with the norm before it run by the norm kernel again)
        return False
    return fills


def _decode_kernel(rows: int, n: int, k: int, mode: str, device) -> str:
    """Which of the two decode kernels takes a product of at most 128 rows: "stream" or "tcgen05"."""
    force = ops.tuning().decode_gemm
    if force == "stream":
        return "stream" if rows <= ops.STREAM_MAX_ROWS else "tcgen05"
    if force == "tcgen05" or rows > STREAM_ROWS:
        return "tcgen05"
    sms = ops.device_state(device)[2]
    return "tcgen05" if tcgen05_for_few_rows(sms, rows, n, k, mode) else "stream"


def _product(out, x, weight, mode: str, up_rows: int = 0) -> None:
    rows = x.shape[0]
    if rows > ops.DECODE_TCGEN05_MAX_ROWS:
        ops.gemm_tcgen05(out, x, weight, mode, up_rows)
    elif _decode_kernel(rows, out.shape[1], x.shape[1], mode, x.device) == "stream":
        ops.gemm_stream(out, x, weight, mode, up_rows)
    else:
        ops.gemm_decode_tcgen05(out, x, weight, mode, up_rows)


def takes_pending(rows: int, n: int, k: int, mode: str, device) -> bool:
    """Whether the product before one of these sizes should prepare its input's norm instead of a norm
    kernel: where the tcgen05 kernels take the product, and where the cp.async kernel takes a plain
    ("store") product (whole steps at a width of 4,096 with q/k/v on it: 1 / 2 / 4 / 8 sequences 3.11 -> 3.09,
    3.20 -> 3.17, 3.43 -> 3.40, 3.79 -> 3.77 ms).  Its SwiGLU product has thousands of short-lived blocks that
    would each add up the parts of the rows' sums of squares before their first product: there the norm
    kernel stays (``ops.Tuning.pending_norm`` = "force" chooses the product all the same)."""
    wish = ops.tuning().pending_norm
    if k % 8 or wish == "off":
        return False
    if rows > ops.DECODE_TCGEN05_MAX_ROWS or wish == "force":
        return True
    return _decode_kernel(rows, n, k, mode, device) == "tcgen05" or mode == "store"


def run_pending(out, pending, weight, up_rows: int = 0) -> None:
    """out = the product of a pending norm's result with weight^T (SwiGLU with ``up_rows``)."""
    rows = pending.shape[0]
    mode = "swiglu" if up_rows else "store"
    if rows > ops.DECODE_TCGEN05_MAX_ROWS:
        kernel = ops.gemm_tcgen05
    elif _decode_kernel(rows, out.shape[1], pending.scaled.shape[1], mode, out.device) == "stream":
        kernel = ops.gemm_stream
    else:
        kernel = ops.gemm_decode_tcgen05
    kernel(out, pending.scaled, weight, mode, up_rows, squares=pending.squares, eps=pending.eps)


def run_with_norm(out, x, weight, norm):
    """out += x . weight^T, and the RMSNorm ``norm`` of the new out prepared on the way: a PendingNorm,
    or None when the kernel that takes this product cannot do that (the caller then runs it plainly)."""
    from .norm import PendingNorm, RMSNorm
    rows, n, k = x.shape[0], out.shape[1], x.shape[1]
    wish = ops.tuning().pending_norm
    if (not isinstance(norm, RMSNorm) or norm.width != n or not aligned(x, weight) or not out.is_contiguous()
            or wish == "off"):
        return None
    by_four = n % 4 == 0 and norm.weight.data_ptr() % 16 == 0  # what the tcgen05 kernels' vector stores need
    if rows > ops.DECODE_TCGEN05_MAX_ROWS:  # a prompt: the tiled tcgen05 product
        if not by_four:
            return None
        kernel, parts = ops.gemm_tcgen05, ops.gemm_tcgen05_norm_parts(n)
    else:
        choice = _decode_kernel(rows, n, k, "accumulate", x.device)
        if wish == "force" and rows <= ops.STREAM_NORM_MAX_ROWS:
            choice = "stream"
        if choice == "stream":
            if rows > ops.STREAM_NORM_MAX_ROWS:
                return None
            kernel, parts = ops.gemm_stream, ops.gemm_stream_norm_parts(rows, n)
        else:  # the few-row tcgen05 product prepares a norm where its splits of K run as clusters
            kernel, parts = ops.gemm_decode_tcgen05, ops.gemm_decode_tcgen05_norm_parts(rows, n, k, x.device)
            if parts == 0 or not by_four:
                return None
    scaled = torch.empty((rows, n), dtype=torch.bfloat16, device=x.device)
    squares = torch.empty((parts, rows), dtype=torch.float32, device=x.device)
    kernel(out, x, weight, "accumulate", norm=(scaled, norm.weight, squares))
    return PendingNorm(scaled, squares, norm.eps, norm)


def run(out, x, weight, accumulate: bool) -> bool:
    if not aligned(x, weight):
        return False
    _product(out, x, weight, "accumulate" if accumulate else "store")
    return True


def run_swiglu(out, x, weight_gate_up, inner: int) -> bool:
    """out = silu(x . gate^T) * (x . up^T) for the fused weight [2 * inner, width]; False if no
    fused kernel takes the shape."""
    from .norm import PendingNorm
    if isinstance(x, PendingNorm):
        run_pending(out, x, weight_gate_up, inner)
        return True
    if not aligned(x, weight_gate_up):
        return False
    _product(out, x, weight_gate_up, "swiglu", inner)
    return True
