"""SwiGLU feed-forward: down( silu(gate(h)) * up(h) ), added to the residual
(crates/xrt-models/src/llama.rs:584-601; crates/xrt-kernels/src/cpu/silu.rs:1-3, 22-24)."""
from __future__ import annotations

import torch

from ..core import DType, torch_dtype
from ..csrc import ops
from .linear import linear
from .registry import register_part


class SwiGLUFeedForward:
    """params: ``width``, ``inner`` (the feed-forward width).
    weights: ``gate``, ``up`` [inner, width], ``down`` [width, inner]."""

    graph_safe = True

    @classmethod
    def fused_weights(cls, params):
        """gate and up are one matrix [gate rows, up rows] for one product."""
        return {"gate_up": ("gate", "up")}

    @classmethod
    def weight_shapes(cls, params):
        d, f = params["width"], params["inner"]
        return {"gate": ((f, d), "matrix"), "up": ((f, d), "matrix"), "down": ((d, f), "matrix")}

    def __init__(self, params, weights, dtype: DType, device):
        self.width = int(params["width"])
        self.inner = int(params["inner"])
        # one fused weight [2 * inner, width]: gate rows, then up rows
        self.w_gate_up = weights.get("gate_up")
        if self.w_gate_up is None:  # tensors that came one by one
            self.w_gate_up = torch.cat([weights["gate"], weights["up"]], dim=0).contiguous()
        self.w_down = weights["down"]
        self.act_dtype = torch_dtype(dtype)

    def takes_pending_norm(self, rows: int, device) -> bool:
        """Whether the first product of ``forward`` can finish a norm that the part before prepared."""
        if self.act_dtype != torch.bfloat16:
            return False
        from . import linear_bf16
        return linear_bf16.takes_pending(rows, self.inner, self.width, "swiglu", device)

    def forward(self, h, residual, ctx):
        act = torch.empty((h.shape[0], self.inner), dtype=self.act_dtype, device=h.device)
        fused = False
        if self.act_dtype == torch.bfloat16 and h.dtype == torch.bfloat16:
            from . import linear_bf16
            fused = linear_bf16.run_swiglu(act, h, self.w_gate_up, self.inner)
        if not fused:
            gate_up = linear(h, self.w_gate_up, out_dtype=torch.float32)
            ops.swiglu(act, gate_up)
        # the last product may prepare the norm that follows this part (ctx.then_norm, see parts/context.py)
        if getattr(ctx, "then_norm", None) is not None:
            _, ctx.pending = linear(act, self.w_down, accumulate_into=residual, then_norm=ctx.then_norm)
        else:
            linear(act, self.w_down, accumulate_into=residual)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
