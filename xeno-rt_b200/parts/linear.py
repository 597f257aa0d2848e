"""y = x . W^T for a weight stored [out, in] as the reference stores every matrix
(crates/xrt-models/src/llama.rs:447-486, no bias anywhere).  Chooses the kernel by dtype and size."""
from __future__ import annotations

import torch

from ..core import KernelError
from ..csrc import ops


def linear(x, weight: torch.Tensor, out_dtype=None, accumulate_into: torch.Tensor | None = None, then_norm=None):
    """Returns x . weight^T in ``out_dtype`` (default float32), or, with ``accumulate_into`` (a
    float32 tensor [M, N], the residual stream), adds the product into it in place and returns it.
    Accumulation is 32-bit in every kernel.  ``x`` may be a ``PendingNorm`` (see parts/norm.py).
    ``then_norm`` (an RMSNorm part, with ``accumulate_into``): if the kernel that runs can prepare that
    norm of the new residual on its way, the result is (residual, PendingNorm), else (residual, None)."""
    from .norm import PendingNorm
    if isinstance(x, PendingNorm):
        from . import linear_bf16
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype or torch.float32, device=x.device)
        linear_bf16.run_pending(out, x, weight)
        return out
    m = x.shape[0]
    n = weight.shape[0]
    if accumulate_into is not None:
        out = accumulate_into
        if out.dtype != torch.float32:
            raise KernelError("linear: the residual stream must be float32")
    else:
        out = torch.empty((m, n), dtype=out_dtype or torch.float32, device=x.device)
    accumulate = accumulate_into is not None
    pending = None
    if m > 0:
        done = False
        if weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16:
            from . import linear_bf16
            if accumulate and then_norm is not None:
                pending = linear_bf16.run_with_norm(out, x, weight, then_norm)
                done = pending is not None
            done = done or linear_bf16.run(out, x, weight, accumulate)
        if not done:
            ops.gemm_reference(out, x, weight, accumulate=accumulate)
    return (out, pending) if then_norm is not None else out
