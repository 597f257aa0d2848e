"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, statistics in 32-bit
(crates/xrt-kernels/src/cpu/rmsnorm.rs:26-43)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..core import torch_dtype
from ..csrc import ops
from .registry import register_part


@dataclass
class PendingNorm:
    """A norm's result that exists only up to its last step: ``scaled`` is the residual times the
    norm's weight (bfloat16 [rows, width]) and ``squares`` (float32 [parts, rows]) holds partial sums
    of squares of the residual's rows, both written by the product that added into the residual.  The
    product that takes this as its input multiplies row m of its result by
    1 / sqrt(sum of the row's parts / width + eps), since W . ((x * inv) * w) = inv * (W . (x * w)):
    no norm kernel runs between the two products of a decode step.  ``norm`` is the part whose result
    this stands for."""
    scaled: torch.Tensor
    squares: torch.Tensor
    eps: float
    norm: object

    @property
    def shape(self):
        return self.scaled.shape

    @property
    def dtype(self):
        return self.scaled.dtype

    @property
    def device(self):
        return self.scaled.device


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
