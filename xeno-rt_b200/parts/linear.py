"""y = x . W^T for a weight stored [out, in] as the reference stores every matrix
(crates/xrt-models/src/llama.rs:447-486, no bias anywhere).  Chooses the kernel by dtype and size."""
from __future__ import annotations

import torch

from ..core import KernelError
from ..csrc import ops


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype=None, accumulate_into: torch.Tensor | None = None):
    """Returns x . weight^T in ``out_dtype`` (default float32), or, with ``accumulate_into`` (a
    float32 tensor [M, N], the residual stream), adds the product into it in place and returns it.
    Accumulation is 32-bit in every kernel."""
    m = x.shape[0]
    n = weight.shape[0]
    if accumulate_into is not None:
        out = accumulate_into
        if out.dtype != torch.float32:
            raise KernelError("linear: the residual stream must be float32")
    else:
        out = torch.empty((m, n), dtype=out_dtype or torch.float32, device=x.device)
    if m == 0:
        return out
    accumulate = accumulate_into is not None
    if weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16:
        from . import linear_bf16
        if linear_bf16.run(out, x, weight, accumulate):
            return out
    ops.gemm_reference(out, x, weight, accumulate=accumulate)
    return out
