"""Rotary position encoding.

The divisor table f_i = base^(2i / rope_dim) is computed once in float32 as the reference does
(crates/xrt-kernels/src/cpu/rope.rs:10-16); each step computes (cos, sin) of
pos * scale / f_i in 32-bit for the step's tokens (rope.rs:59-68).  The rotation itself is applied
by the attention mixer's fused kernel from this table, so any encoding that is a rotation of pairs
of a head's dims by position-dependent angles fits this interface by returning another table.  A
position part says which dims pair up with ``pairing``: "split_half" (i with i + rope_dim / 2, the
reference's and the default, rope.rs:19-35) or "interleaved" (2i with 2i + 1); dims from rope_dim on
stay as they are (rope.rs:19-35 rotates ``rope_dim`` dims of each head only).
"""
from __future__ import annotations

import numpy as np
import torch

from ..core import ConfigError
from ..csrc import ops
from .registry import register_part


class RotaryEncoding:
    """params: ``rope_dim`` (even, at most the head size), ``base``, ``scale`` (multiplies the
    position), ``pairing`` ("split_half" or "interleaved").  No weights."""

    @classmethod
    def weight_shapes(cls, params):
        return {}

    def __init__(self, params, weights, dtype, device):
        self.rope_dim = int(params["rope_dim"])
        self.base = float(params["base"])
        self.scale = float(params.get("scale", 1.0))
        self.pairing = str(params.get("pairing", "split_half"))
        if self.rope_dim <= 0 or self.rope_dim % 2:
            raise ConfigError(f"rope_dim {self.rope_dim} must be a positive even number")
        if self.pairing not in ("split_half", "interleaved"):
            raise ConfigError(f"pairing {self.pairing!r} is not split_half or interleaved")
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

    pairing = "split_half"

    @classmethod
    def weight_shapes(cls, params):
        return {}

    def __init__(self, params, weights, dtype, device):
        pass

    def tables(self, ctx):
        return None


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
