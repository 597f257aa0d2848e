"""The Llama / Qwen3 dense decoder of the reference (crates/xrt-models/src/llama.rs): pre-norm
residual blocks with RMSNorm, grouped-query attention with split-half rotary encoding, optional
per-head q/k RMSNorm (Qwen3), SwiGLU feed-forward, final RMSNorm, tied or untied output matrix.

The reference reads the configuration from GGUF metadata (llama.rs:41-137); this module reads the
same quantities from the config.json keys of the two architectures and names tensors as their
safetensors files do.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..config import ModelConfig, register_architecture
from ..config.base import KeyReader
from ..core import Unsupported
from ..parts import ModelSpec, PartSpec, SchedulePlace, prenorm_layer


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    """Sizes and constants of one Llama / Qwen3 model.  Defaults follow llama.rs:41-137:
    kv heads = heads (68-70), head size = hidden / heads unless given (76-80, 125-128),
    eps 1e-5 (95-98), rope base 10000 (99-102), rope scale 1 (103-106)."""
    architecture: str
    vocab_size: int
    max_position_embeddings: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scale: float
    tie_word_embeddings: bool
    qk_norm: bool
    eos_token_ids: tuple
    torch_dtype: str

    DEFAULT_EPS = 1e-5
    QK_NORM = False

    @classmethod
    def from_dict(cls, raw: dict) -> "LlamaConfig":
        r = KeyReader(raw)
        arch = raw["architectures"][0]
        vocab = r.positive_int("vocab_size")
        max_pos = r.positive_int("max_position_embeddings")
        hidden = r.positive_int("hidden_size")
        inner = r.positive_int("intermediate_size")
        layers = r.positive_int("num_hidden_layers")
        heads = r.positive_int("num_attention_heads")
        kv_heads = r.positive_int("num_key_value_heads", default=heads)
        head_dim = r.positive_int("head_dim", default=(hidden // heads if hidden and heads else None))
        eps = r.number("rms_norm_eps", default=cls.DEFAULT_EPS)
        theta = r.number("rope_theta", default=10000.0)
        tied = r.boolean("tie_word_embeddings", default=False)
        if heads and kv_heads and heads % kv_heads:
            r.fail(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if "head_dim" not in raw and hidden and heads and hidden % heads:
            r.fail(f"hidden_size {hidden} is not a multiple of num_attention_heads {heads} and no head_dim is given")
        if head_dim and head_dim % 2:
            r.fail(f"head_dim {head_dim} must be even for the rotary encoding")
        r.finish()
        if raw.get("rope_scaling") not in (None, {}):
            raise Unsupported(f"config.json: rope_scaling {raw['rope_scaling']!r} is not supported (only none)")
        for key in ("attention_bias", "mlp_bias"):
            if raw.get(key):
                raise Unsupported(f"config.json: {key} = true is not supported; the architecture has no biases")
        if raw.get("hidden_act", "silu") != "silu":
            raise Unsupported(f"config.json: hidden_act {raw['hidden_act']!r} is not supported; the feed-forward of "
                              f"this architecture is SiLU-gated (crates/xrt-kernels/src/cpu/silu.rs:1-3)")
        if raw.get("partial_rotary_factor") not in (None, 1, 1.0):
            raise Unsupported(f"config.json: partial_rotary_factor {raw['partial_rotary_factor']!r} is not supported; "
                              f"this architecture rotates all of a head")
        if raw.get("use_sliding_window"):
            raise Unsupported("config.json: use_sliding_window = true is not supported by this architecture")
        return cls(architecture=arch, vocab_size=vocab, max_position_embeddings=max_pos, hidden_size=hidden,
                   intermediate_size=inner, num_hidden_layers=layers, num_attention_heads=heads,
                   num_key_value_heads=kv_heads, head_dim=head_dim, rms_norm_eps=eps, rope_theta=theta,
                   rope_scale=1.0, tie_word_embeddings=tied, qk_norm=cls.QK_NORM,
                   eos_token_ids=r.int_tuple("eos_token_id"), torch_dtype=str(raw.get("torch_dtype", "bfloat16")))

    def to_dict(self) -> dict:
        out = {"architectures": [self.architecture], "vocab_size": self.vocab_size,
               "max_position_embeddings": self.max_position_embeddings, "hidden_size": self.hidden_size,
               "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
               "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
               "head_dim": self.head_dim, "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
               "rope_scaling": None, "tie_word_embeddings": self.tie_word_embeddings,
               "attention_bias": False, "mlp_bias": False, "hidden_act": "silu", "torch_dtype": self.torch_dtype}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out

    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim


@dataclass(frozen=True)
class Qwen3Config(LlamaConfig):
    """Qwen3 is the same decoder with per-head q/k RMSNorm (llama.rs:313-336, 488-496) and eps
    1e-6 as its configurations write it."""
    DEFAULT_EPS = 1e-6
    QK_NORM = True


def build_spec(cfg: LlamaConfig) -> ModelSpec:
    """One LayerSpec for each of the model's layers, run once each in order."""
    d, eps = cfg.hidden_size, cfg.rms_norm_eps
    position = {"kind": "rotary", "params": {"rope_dim": cfg.head_dim, "base": cfg.rope_theta,
                                             "scale": cfg.rope_scale}}
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        attn_weights = {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                        "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"}
        if cfg.qk_norm:
            attn_weights["q_norm"] = p + "self_attn.q_norm.weight"
            attn_weights["k_norm"] = p + "self_attn.k_norm.weight"
        layers.append(prenorm_layer(
            mixer_norm=PartSpec("rmsnorm", {"width": d, "eps": eps}, {"weight": p + "input_layernorm.weight"}),
            mixer=PartSpec("attention", {"width": d, "n_heads": cfg.num_attention_heads,
                                         "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                                         "qk_norm": cfg.qk_norm, "eps": eps, "window": None,
                                         "position": position}, attn_weights),
            ffn_norm=PartSpec("rmsnorm", {"width": d, "eps": eps},
                              {"weight": p + "post_attention_layernorm.weight"}),
            ffn=PartSpec("swiglu", {"width": d, "inner": cfg.intermediate_size},
                         {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                          "down": p + "mlp.down_proj.weight"})))
    head_name = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=d, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token", {"vocab_size": cfg.vocab_size, "width": d},
                           {"weight": "model.embed_tokens.weight"}),
        layers=layers,
        schedule=[SchedulePlace(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"width": d, "eps": eps}, {"weight": "model.norm.weight"}),
        lm_head=PartSpec("linear", {"vocab_size": cfg.vocab_size, "width": d}, {"weight": head_name}),
        stop_ids=tuple(cfg.eos_token_ids),
        ignorable_tensors=("*.rotary_emb.inv_freq",))


register_architecture("LlamaForCausalLM", LlamaConfig, build_spec)
register_architecture("Qwen3ForCausalLM", Qwen3Config, build_spec)
