"""Rotary position encoding with split-half pairing.

The divisor table f_i = base^(2i / rope_dim) is computed once in float32 as the reference does
(crates/xrt-kernels/src/cpu/rope.rs:10-16); each step computes (cos, sin) of
pos * scale / f_i in 32-bit for the step's tokens (rope.rs:59-68).  The rotation itself is applied
by the attention mixer's fused kernel from this table, so any encoding that is a rotation of
(i, i + half) pairs by position-dependent angles fits this interface by returning another table.
"""
from __future__ import annotations

import numpy as np
import torch

from ..csrc import ops
from .registry import register_part


class RotaryEncoding:
    """params: ``rope_dim`` (even, at most the head size), ``base``, ``scale`` (multiplies the
    position).  No weights."""

    @classmethod
    def weight_shapes(cls, params):
        return {}

    def __init__(self, params, weights, dtype, device):
        self.rope_dim = int(params["rope_dim"])
        self.base = float(params["base"])
        self.scale = float(params.get("scale", 1.0))
        self.half = self.rope_dim // 2
        i = np.arange(self.half, dtype=np.float32)
        freq = np.power(np.float32(self.base), (np.float32(2.0) * i) / np.float32(self.rope_dim)).astype(np.float32)
        self.freq = torch.from_numpy(freq).to(device)
        self._key = ("rotary", self.rope_dim, self.base, self.scale)

    def tables(self, ctx):
        """(cos, sin) float32 [T, half, 2] for the tokens of the step; computed once a step."""
        table = ctx.shared.get(self._key)
        if table is None:
            table = torch.empty((ctx.n_tokens, self.half, 2), dtype=torch.float32, device=self.freq.device)
            ops.rope_table(table, ctx.tok_pos, self.freq, self.scale)
            ctx.shared[self._key] = table
        return table


class NoPositionEncoding:
    """Leaves q and k as they are."""

    @classmethod
    def weight_shapes(cls, params):
        return {}

    def __init__(self, params, weights, dtype, device):
        pass

    def tables(self, ctx):
        return None


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
