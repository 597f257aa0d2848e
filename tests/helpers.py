"""Shared fixtures of the tests: two tiny configurations that differ in every size and option,
model folders made in temporary directories, and comparison helpers."""
from __future__ import annotations

import json
import os

import numpy as np

# Differ in: architecture, stored dtype, layers, width, heads, kv heads (group 2 vs 3), head size
# (width = heads * head size in one, not in the other), feed-forward width (no power of two),
# vocabulary (a power of two vs not), positions, rope base, eps, q/k norm, tied output.
TINY_LLAMA = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 256, "max_position_embeddings": 128,
    "hidden_size": 64, "intermediate_size": 176, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "eos_token_id": 7,
}
TINY_QWEN3 = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 320, "max_position_embeddings": 256,
    "hidden_size": 96, "intermediate_size": 160, "num_hidden_layers": 3, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 32, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "eos_token_id": [3, 11],
}
# A third one for the long and odd cases: width and vocabulary that are no multiple of 8, head
# size 48, one kv head for five heads, many positions.
TINY_ODD = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 203, "max_position_embeddings": 1024,
    "hidden_size": 100, "intermediate_size": 136, "num_hidden_layers": 2, "num_attention_heads": 5,
    "num_key_value_heads": 1, "head_dim": 48, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False,
}
# A fourth one with the head size of the large models, so that whole-model runs reach the kernels
# that only take it: the tcgen05 prompt attention, the decode attention fed by TMA, and (with a
# prompt of more than 128 tokens) the tiled tcgen05 product.
TINY_WIDE = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 520, "max_position_embeddings": 1024,
    "hidden_size": 256, "intermediate_size": 384, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 128, "rope_theta": 20000.0, "rms_norm_eps": 2e-5,
    "tie_word_embeddings": False,
}
CONFIGS = {"tiny-llama": (TINY_LLAMA, 0, "float32"), "tiny-qwen3": (TINY_QWEN3, 1, "bfloat16"),
           "tiny-odd": (TINY_ODD, 2, "bfloat16"), "tiny-wide": (TINY_WIDE, 3, "bfloat16")}


def make_folder(tmp_path, name: str, sharpen: float = 1.0) -> str:
    """Writes the named tiny model with the library's random-weights mode.  ``sharpen`` > 1 scales
    the q and k matrices so that attention scores spread out and a wrong key shows in the result
    (with N(0, 0.02) weights every softmax is almost uniform and would hide it)."""
    from xeno_rt_b200.weights import read_safetensors, write_random_model, write_safetensors

    raw, seed, dtype = CONFIGS[name]
    folder = os.path.join(str(tmp_path), name + (f"-sharp{sharpen}" if sharpen != 1.0 else ""))
    write_random_model(folder, raw, seed, dtype)
    if sharpen != 1.0:
        path = os.path.join(folder, "model.safetensors")
        tensors = read_safetensors(path)
        for key in tensors:
            if key.endswith("q_proj.weight") or key.endswith("k_proj.weight"):
                tensors[key] = (tensors[key].float() * sharpen).to(tensors[key].dtype)
        write_safetensors(path, tensors)
    return folder


def random_prompts(vocab: int, lengths, seed: int = 0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]


def scaled_error(got: np.ndarray, want: np.ndarray) -> float:
    """Largest absolute difference relative to the largest wanted magnitude (the logit scale)."""
    return float(np.abs(got.astype(np.float64) - want).max() / np.abs(want).max())


# Tolerances, relative to the logit scale.  32-bit: the kernels sum in another order than the
# float64 oracle.  bfloat16: activations are rounded to 8 bits of mantissa at the inputs of every
# matrix product and in the cache.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def check_greedy_tokens(plain_config, plain_weights, prompt, tokens, tolerance: float):
    """Greedy tokens of the engine against the plain model along the engine's own path: the plain
    logits of prompt + tokens (teacher-forced) say, at every generated place, which token is best
    and by how much.  Where the two best logits lie further apart than twice the tolerance (of the
    logit scale), the engine's token must be the best one; at a nearer tie either may win, and from
    there on the engine's continuation is judged along its own path, not dropped.  Returns the plain
    logits [len(prompt) + len(tokens), vocab]."""
    from plain.model import forward_logits

    want = forward_logits(plain_config, plain_weights, list(prompt) + list(tokens))
    scale = np.abs(want).max()
    for i, token in enumerate(tokens):
        row = want[len(prompt) + i - 1]
        top = np.sort(row)[-2:]
        if top[1] - top[0] > 2 * tolerance * scale:
            assert int(token) == int(np.argmax(row)), (list(prompt), i, int(token), int(np.argmax(row)))
    return want


def replay_logits(engine, prompt, tokens):
    """Logits of every place of prompt + tokens through ``engine.step``: the prompt in one step, then
    one token a step."""
    from xeno_rt_b200.engine import StepEntry
    slot = engine.open_slot()
    rows = [engine.step([StepEntry(slot, list(prompt), list(range(len(prompt))))]).cpu().numpy()]
    rows += [engine.step([StepEntry(slot, [int(t)], [0])]).cpu().numpy() for t in tokens]
    engine.close_slot(slot)
    return np.concatenate(rows)
