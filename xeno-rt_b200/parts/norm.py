"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, statistics in 32-bit
(crates/xrt-kernels/src/cpu/rmsnorm.rs:26-43)."""
from __future__ import annotations

import torch

from ..core import torch_dtype
from ..csrc import ops
from .registry import register_part


class RMSNorm:
    """params: ``width``, ``eps``.  weights: ``weight`` [width]."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["width"],), "vector")}

    def __init__(self, params, weights, dtype, device):
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.weight = weights["weight"]
        self.out_dtype = torch_dtype(dtype)

    def forward(self, x, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=self.out_dtype, device=x.device)
        ops.rmsnorm(out, x, self.weight, self.eps, rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
