"""Plain, slow restatement of the Llama / Qwen3 dense decoder, one function per part.

This file is the oracle of the test-suite.  It shares no code with the product
package: it has its own safetensors reader (``tests/plain/files.py``), works on
whole sequences without any cache, and uses numpy float64 arithmetic so that
its own rounding never decides a comparison.

It rests on the formulas of the reference project only (its Rust sources cannot
be compiled where these tests run: there is no Rust toolchain, and the
reference model accepts GGUF-quantised matrices only).  Every function cites the
file and lines of the reference it restates; paths are relative to the
reference project root.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


def embedding(table: np.ndarray, token_ids) -> np.ndarray:
    """x = E[token]; an id outside the table is an error, there is no scaling.

    crates/xrt-models/src/llama.rs:1042-1055 (embedding_lookup), used at 432.
    """
    ids = np.asarray(token_ids, dtype=np.int64)
    if ids.size and (ids.min() < 0 or ids.max() >= table.shape[0]):
        raise ValueError("token id outside the embedding table")
    return table[ids].astype(F64)


def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """y = (x * 1/sqrt(mean(x^2) + eps)) * w, the weight multiplies directly.

    crates/xrt-kernels/src/cpu/rmsnorm.rs:26-43 (mean square, inv_rms, product).
    Works on the last axis, so it also serves the per-head q/k norm.
    """
    x = x.astype(F64)
    mean_square = np.mean(x * x, axis=-1, keepdims=True)
    inv_rms = 1.0 / np.sqrt(mean_square + F64(eps))
    return (x * inv_rms) * weight.astype(F64)


def linear(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    """y = W x with W stored [out, in] row-major, no bias anywhere.

    crates/xrt-models/src/llama.rs:447-486 (q, k, v), 576 (o), 584-599 (mlp).
    """
    return x.astype(F64) @ weight.astype(F64).T


def head_rmsnorm(x: np.ndarray, weight: np.ndarray, n_heads: int, head_dim: int, eps: float) -> np.ndarray:
    """RMSNorm over each head slice with one weight [head_dim] for all heads.

    crates/xrt-models/src/llama.rs:1025-1040 (apply_head_norm), called at 488-496
    after the projection and before the rotation, with the model's eps.
    """
    t = x.shape[0]
    heads = x.reshape(t, n_heads, head_dim)
    return rmsnorm(heads, weight, eps).reshape(t, n_heads * head_dim)


def rope_frequencies(rope_dim: int, base: float) -> np.ndarray:
    """f_i = base^(2i / rope_dim), stored as the divisor of the angle, in float32.

    crates/xrt-kernels/src/cpu/rope.rs:10-16 (RopeFreqs::new uses f32 powf).
    """
    half = rope_dim // 2
    i = np.arange(half, dtype=np.float32)
    return np.power(np.float32(base), (np.float32(2.0) * i) / np.float32(rope_dim)).astype(np.float32)


def rope(x: np.ndarray, positions, n_heads: int, head_dim: int, rope_dim: int, base: float,
         scale: float, pairing: str = "split_half") -> np.ndarray:
    """Split-half rotation of every head at the token's absolute position.

    angle = pos * scale / f_i in float32 (as the reference computes it), then
    h[i]      = x0 * cos - x1 * sin
    h[i+half] = x0 * sin + x1 * cos      with x0 = h[i], x1 = h[i + half].
    Elements at or beyond rope_dim stay as they are.
    crates/xrt-kernels/src/cpu/rope.rs:19-35 (apply), 59-68 (angles).
    ``pairing`` = "interleaved" is not the reference's: x0 = h[2i], x1 = h[2i + 1] with the same
    angles, for the library's position encodings that pair neighbouring dims.
    """
    t = x.shape[0]
    half = min(rope_dim, head_dim) // 2
    freqs = rope_frequencies(rope_dim, base)[:half]
    pos = np.asarray(positions, dtype=np.float32).reshape(t, 1)
    angle = (pos * np.float32(scale) / freqs.reshape(1, half)).astype(np.float32).astype(F64)
    sin, cos = np.sin(angle), np.cos(angle)
    heads = x.astype(F64).reshape(t, n_heads, head_dim).copy()
    first = slice(0, 2 * half, 2) if pairing == "interleaved" else slice(0, half)
    second = slice(1, 2 * half, 2) if pairing == "interleaved" else slice(half, 2 * half)
    x0 = heads[:, :, first].copy()
    x1 = heads[:, :, second].copy()
    heads[:, :, first] = x0 * cos[:, None, :] - x1 * sin[:, None, :]
    heads[:, :, second] = x0 * sin[:, None, :] + x1 * cos[:, None, :]
    return heads.reshape(t, n_heads * head_dim)


def softmax(scores: np.ndarray) -> np.ndarray:
    """Max-subtracted softmax over the last axis.

    crates/xrt-kernels/src/cpu/softmax.rs:14-40 (scalar form).
    """
    m = np.max(scores, axis=-1, keepdims=True)
    e = np.exp(scores - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def causal_gqa_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, n_heads: int, n_kv_heads: int,
                         head_dim: int, window: int | None = None) -> np.ndarray:
    """Full causal attention of one whole sequence that starts at position 0.

    Query head h reads kv head h // (n_heads / n_kv_heads); the scale is
    1/sqrt(head_dim); the causal mask is the bound j <= t of the key loop.
    crates/xrt-models/src/llama.rs:728-770 (prefill form), 504-574 (decode form).
    ``window`` (absent in the reference) keeps keys with t - j < window.
    """
    t = q.shape[0]
    group = n_heads // n_kv_heads
    scale = 1.0 / math.sqrt(head_dim)
    qh = q.astype(F64).reshape(t, n_heads, head_dim)
    kh = k.astype(F64).reshape(t, n_kv_heads, head_dim)
    vh = v.astype(F64).reshape(t, n_kv_heads, head_dim)
    out = np.zeros((t, n_heads, head_dim), dtype=F64)
    for h in range(n_heads):
        kv = h // group
        for i in range(t):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (kh[lo:i + 1, kv, :] @ qh[i, h, :]) * scale
            p = softmax(s)
            out[i, h, :] = p @ vh[lo:i + 1, kv, :]
    return out.reshape(t, n_heads * head_dim)


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """a_i = (g_i / (1 + exp(-g_i))) * u_i.

    crates/xrt-kernels/src/cpu/silu.rs:1-3, 22-24.
    """
    g = gate.astype(F64)
    return (g / (1.0 + np.exp(-g))) * up.astype(F64)


def attention_block(x, w, prefix, cfg, positions):
    """normed -> q, k, v -> (head norms) -> rotation -> attention -> o-projection.

    crates/xrt-models/src/llama.rs:441-577.
    """
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = linear(x, w[prefix + "self_attn.q_proj.weight"])
    k = linear(x, w[prefix + "self_attn.k_proj.weight"])
    v = linear(x, w[prefix + "self_attn.v_proj.weight"])
    if cfg["qk_norm"]:
        q = head_rmsnorm(q, w[prefix + "self_attn.q_norm.weight"], nh, hd, eps)
        k = head_rmsnorm(k, w[prefix + "self_attn.k_norm.weight"], nkv, hd, eps)
    q = rope(q, positions, nh, hd, hd, cfg["rope_theta"], cfg["rope_scale"])
    k = rope(k, positions, nkv, hd, hd, cfg["rope_theta"], cfg["rope_scale"])
    o = causal_gqa_attention(q, k, v, nh, nkv, hd)
    return linear(o, w[prefix + "self_attn.o_proj.weight"])


def mlp_block(x, w, prefix):
    """gate, up -> SwiGLU -> down.  crates/xrt-models/src/llama.rs:584-599."""
    gate = linear(x, w[prefix + "mlp.gate_proj.weight"])
    up = linear(x, w[prefix + "mlp.up_proj.weight"])
    return linear(swiglu(gate, up), w[prefix + "mlp.down_proj.weight"])


def decoder_block(x, w, layer, cfg, positions):
    """x + Attn(RMSNorm(x)), then x + MLP(RMSNorm(x)).  llama.rs:433-602."""
    prefix = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    x = x + attention_block(rmsnorm(x, w[prefix + "input_layernorm.weight"], eps), w, prefix, cfg, positions)
    x = x + mlp_block(rmsnorm(x, w[prefix + "post_attention_layernorm.weight"], eps), w, prefix)
    return x


def normalise_config(raw: dict) -> dict:
    """The keys this file needs, with the defaults of llama.rs:41-137 restated for config.json."""
    arch = raw["architectures"][0]
    cfg = dict(raw)
    cfg.setdefault("num_key_value_heads", raw["num_attention_heads"])
    cfg.setdefault("head_dim", raw["hidden_size"] // raw["num_attention_heads"])
    cfg.setdefault("rms_norm_eps", 1e-5)
    cfg.setdefault("rope_theta", 10000.0)
    cfg.setdefault("tie_word_embeddings", False)
    cfg["rope_scale"] = 1.0
    cfg["qk_norm"] = arch == "Qwen3ForCausalLM"
    return cfg


def forward_logits(raw_config: dict, weights: dict, token_ids) -> np.ndarray:
    """Logits [T, vocab] at every position of one whole sequence from position 0.

    crates/xrt-models/src/llama.rs:830-1009 (forward_batch_all_logits): the
    blocks in order, the final norm, the output matrix (the embedding if tied,
    llama.rs:301-305).
    """
    cfg = normalise_config(raw_config)
    positions = np.arange(len(token_ids))
    x = embedding(weights["model.embed_tokens.weight"], token_ids)
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_block(x, weights, layer, cfg, positions)
    x = rmsnorm(x, weights["model.norm.weight"], cfg["rms_norm_eps"])
    head = weights["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else weights["lm_head.weight"]
    return linear(x, head)


def greedy_generate(raw_config: dict, weights: dict, prompt, max_tokens: int, stop_ids=()) -> list[int]:
    """Greedy continuation by re-running the whole sequence for every new token.

    The loop order is that of crates/xrt-runtime/src/session.rs:115-141: sample
    from the current logits, stop on a stop id (not emitted) or a full
    context, append, run again.  argmax keeps the first maximum
    (crates/xrt-runtime/src/sampler.rs:83-98, strict ``>``).
    """
    cfg = normalise_config(raw_config)
    tokens = list(prompt)
    out: list[int] = []
    while len(out) < max_tokens:
        logits = forward_logits(raw_config, weights, tokens)[-1]
        nxt = int(np.argmax(logits))
        if nxt in stop_ids:
            break
        if len(tokens) >= cfg["max_position_embeddings"]:
            break
        tokens.append(nxt)
        out.append(nxt)
    return out
