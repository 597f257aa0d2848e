"""Choice among the bfloat16 attention kernels.  ``run`` returns False when none takes the case,
and the caller uses the kernel that takes any."""
from __future__ import annotations


def run(out, q, ctx, store, n_heads, n_kv_heads, head_dim, scale, window) -> bool:
    return False
