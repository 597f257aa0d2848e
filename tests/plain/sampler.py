"""Plain restatement of the reference's sampler (crates/xrt-runtime/src/sampler.rs).

The random draw ``r`` is an argument: the product uses its own documented
generator, so tests pass the same ``r`` to both sides.
"""
from __future__ import annotations

import numpy as np


def penalised(logits, history, repetition_penalty: float) -> np.ndarray:
    """l > 0 ? l / p : l * p for every id that occurs in the history, if p > 1.

    sampler.rs:77-91 (greedy) and 110-125 (temperature): a set of seen ids, so
    an id that occurs twice is penalised once.
    """
    out = np.asarray(logits, dtype=np.float64).copy()
    if repetition_penalty > 1.0 and len(history):
        for tok in set(int(t) for t in history):
            out[tok] = out[tok] / repetition_penalty if out[tok] > 0 else out[tok] * repetition_penalty
    return out


def greedy(logits, history=(), repetition_penalty: float = 1.0) -> int:
    """First maximum wins (strict >).  sampler.rs:83-98."""
    return int(np.argmax(penalised(logits, history, repetition_penalty)))


def candidate_distribution(logits, history, temperature, top_k, top_p, repetition_penalty):
    """(ids, probabilities) of the kept candidates, sorted by falling logit.

    sampler.rs:107-183: the top_k largest adjusted logits (0 = all; among equal
    values the earlier index is kept), softmax of (l - max) / T over them, then the
    shortest prefix whose cumulative probability reaches top_p, renormalised.
    """
    adj = penalised(logits, history, repetition_penalty)
    n = len(adj)
    k = top_k if top_k > 0 else n
    order = np.argsort(-adj, kind="stable")[:k]
    vals = adj[order]
    probs = np.exp((vals - vals[0]) / temperature)
    probs = probs / probs.sum()
    keep = len(order)
    if top_p < 1.0:
        cum = np.cumsum(probs)
        keep = int(np.searchsorted(cum, top_p, side="left")) + 1
        keep = max(1, min(keep, len(order)))
        probs = probs[:keep] / probs[:keep].sum()
    return order[:keep], probs[:keep]


def sample(logits, r: float, history=(), temperature=0.8, top_k=40, top_p=0.95,
           repetition_penalty=1.1) -> int:
    """sampler.rs:50-69 and 186-195: greedy if T <= 1e-5, else walk the cumulative sum with r <= cum."""
    if temperature <= 1e-5:
        return greedy(logits, history, repetition_penalty)
    ids, probs = candidate_distribution(logits, history, temperature, top_k, top_p, repetition_penalty)
    cum = 0.0
    for idx, p in zip(ids, probs):
        cum += p
        if r <= cum:
            return int(idx)
    return int(ids[0])
