"""Grouped-query causal attention with optional per-head q/k RMSNorm and a position encoding.

Order, as in crates/xrt-models/src/llama.rs:447-577: q, k, v products; per-head norm of q and k if
the layer has one (488-496, 1025-1040); rotation (498-500); k and v into the cache (502); attention of
every query head over the keys of its group's kv head up to its own position with scale
1/sqrt(head_dim) (504-574); output product added to the residual (576-577).
"""
from __future__ import annotations

import math

import torch

from ..cache import KVNeed
from ..core import ConfigError, DType, Unsupported, torch_dtype
from ..csrc import ops
from .linear import linear
from .registry import part_class, register_part


class GroupedQueryAttention:
    """params: ``width`` (model width), ``n_heads``, ``n_kv_heads``, ``head_dim``, ``qk_norm``
    (bool), ``eps`` (of the head norms), ``window`` (None = all keys), ``position`` (a PartSpec-like
    dict ``{"kind", "params"}``).
    weights: ``q`` [n_heads*head_dim, width], ``k``, ``v`` [n_kv_heads*head_dim, width],
    ``o`` [width, n_heads*head_dim], and with qk_norm ``q_norm``, ``k_norm`` [head_dim]."""

    graph_safe = True

    @classmethod
    def fused_weights(cls, params):
        """q, k and v are one matrix [q rows, k rows, v rows] for one product."""
        return {"qkv": ("q", "k", "v")}

    @classmethod
    def weight_shapes(cls, params):
        d, nh, nkv, hd = params["width"], params["n_heads"], params["n_kv_heads"], params["head_dim"]
        shapes = {"q": ((nh * hd, d), "matrix"), "k": ((nkv * hd, d), "matrix"), "v": ((nkv * hd, d), "matrix"),
                  "o": ((d, nh * hd), "matrix")}
        if params.get("qk_norm"):
            shapes["q_norm"] = ((hd,), "vector")
            shapes["k_norm"] = ((hd,), "vector")
        return shapes

    def __init__(self, params, weights, dtype: DType, device):
        self.width = int(params["width"])
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.eps = float(params.get("eps", 1e-5))
        self.window = params.get("window")
        if self.n_heads % self.n_kv_heads:
            raise ConfigError(f"{self.n_heads} heads are not a multiple of {self.n_kv_heads} kv heads")
        if self.head_dim % 16 or not (16 <= self.head_dim <= 256):
            raise Unsupported(f"head size {self.head_dim}: the attention kernels take multiples of 16 up to 256")
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        # one fused weight for the three products; the reference fuses only their dispatch (447-486)
        self.w_qkv = weights.get("qkv")
        if self.w_qkv is None:  # tensors that came one by one
            self.w_qkv = torch.cat([weights["q"], weights["k"], weights["v"]], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.q_width]
        self.w_o = weights["o"]
        self.q_norm = weights.get("q_norm") if params.get("qk_norm") else None
        self.k_norm = weights.get("k_norm") if params.get("qk_norm") else None
        position = params.get("position") or {"kind": "none", "params": {}}
        self.position = part_class("position", position["kind"])(position.get("params", {}), {}, dtype, device)
        rope_dim = getattr(self.position, "rope_dim", 0)
        if rope_dim > self.head_dim:
            raise ConfigError(f"rope_dim {rope_dim} exceeds the head size {self.head_dim}")
        self.scale = 1.0 / math.sqrt(self.head_dim)
        self.dtype = dtype
        self.act_dtype = torch_dtype(dtype)

    def cache_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window)

    def takes_pending_norm(self, rows: int, device) -> bool:
        """Whether the first product of ``forward`` can finish a norm that the part before prepared."""
        if self.dtype is not DType.BF16:
            return False
        from . import linear_bf16
        return linear_bf16.takes_pending(rows, self.w_qkv.shape[0], self.width, "store", device)

    def forward(self, h, residual, ctx, store, owns_cache=True):
        n = h.shape[0]
        then_norm = getattr(ctx, "then_norm", None)  # for this part's last product only
        if then_norm is not None:
            ctx.then_norm = None
        qkv = linear(h, self.w_qkv if owns_cache else self.w_q, out_dtype=torch.float32)
        window = int(self.window) if self.window else 0
        pairing = getattr(self.position, "pairing", "split_half")
        cos_sin = self.position.tables(ctx)
        # padding rows belong to no sequence: kernels that walk sequences leave them unwritten
        padded = sum(ctx.new_lens) < ctx.n_tokens
        attended = (torch.zeros if padded else torch.empty)((n, self.q_width), dtype=self.act_dtype, device=h.device)
        if self.dtype is DType.BF16:
            from . import attention_bf16
            if attention_bf16.decode_from_qkv(attended, qkv, self.q_width, self.q_width + self.kv_width, self.q_norm,
                                              self.k_norm, self.eps, cos_sin, pairing, ctx, store, self.n_heads,
                                              self.n_kv_heads, self.head_dim, self.scale, window, owns_cache):
                qkv = None
        if qkv is not None:
            q = torch.empty((n, self.q_width), dtype=self.act_dtype, device=h.device)
            ops.qk_rope_kv_write(q, store.k, store.v, qkv, self.q_width, self.q_width + self.kv_width, self.q_norm,
                                 self.k_norm, self.eps, cos_sin, ctx.tok_slot, ctx.tok_pos, store.block_table,
                                 self.n_heads, self.n_kv_heads, self.head_dim, write_kv=owns_cache, pairing=pairing)
            self.attend(attended, q, ctx, store)
        if then_norm is not None:
            _, ctx.pending = linear(attended, self.w_o, accumulate_into=residual, then_norm=then_norm)
        else:
            linear(attended, self.w_o, accumulate_into=residual)

    def attend(self, out, q, ctx, store):
        window = int(self.window) if self.window else 0
        if self.dtype is DType.BF16:
            from . import attention_bf16
            if attention_bf16.run(out, q, ctx, store, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                  window):
                return
        ops.attention_reference(out, q, store.k, store.v, ctx.tok_slot, ctx.tok_pos, store.block_table,
                                self.n_heads, self.n_kv_heads, self.head_dim, self.scale, window)


register_part("mixer", "attention", GroupedQueryAttention)
