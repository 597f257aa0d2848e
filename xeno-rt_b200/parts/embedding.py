"""Token embedding and the output matrix."""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import linear
from .registry import register_part


class TokenEmbedding:
    """x = E[token], no scaling (crates/xrt-models/src/llama.rs:1042-1055).
    params: ``vocab_size``, ``width``.  weights: ``weight`` [vocab, width]."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["vocab_size"], params["width"]), "matrix")}

    def __init__(self, params, weights, dtype, device):
        self.vocab_size = int(params["vocab_size"])
        self.width = int(params["width"])
        self.weight = weights["weight"]

    def forward(self, token_ids, error_flag):
        out = torch.empty((token_ids.numel(), self.width), dtype=torch.float32, device=token_ids.device)
        ops.embedding(out, self.weight, token_ids, error_flag)
        return out


class OutputHead:
    """logits = W . normed, no scaling or cap (crates/xrt-models/src/llama.rs:604-613); W is the
    embedding when the model ties them (llama.rs:301-305), which the spec expresses by giving both
    parts the same tensor name.  params: ``vocab_size``, ``width``.  weights: ``weight``."""

    graph_safe = True

    @classmethod
    def weight_shapes(cls, params):
        return {"weight": ((params["vocab_size"], params["width"]), "matrix")}

    def __init__(self, params, weights, dtype, device):
        self.weight = weights["weight"]

    def forward(self, normed):
        return linear(normed, self.weight, out_dtype=torch.float32)


register_part("embedding", "token", TokenEmbedding)
register_part("lm_head", "linear", OutputHead)
