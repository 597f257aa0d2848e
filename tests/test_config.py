"""Configuration and registry (no GPU)."""
import json

import pytest

import xeno_rt_b200  # noqa: F401
from xeno_rt_b200.config import architecture_names, config_from_dict, load_config
from xeno_rt_b200.core import ConfigError, Unsupported
from helpers import TINY_LLAMA, TINY_QWEN3


def test_registry_names():
    assert {"LlamaForCausalLM", "Qwen3ForCausalLM"} <= set(architecture_names())


def test_llama_fields_and_defaults():
    arch, cfg = config_from_dict(TINY_LLAMA)
    assert arch.name == "LlamaForCausalLM"
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (64, 4, 2, 16)
    assert cfg.qk_norm is False and cfg.tie_word_embeddings is False
    assert cfg.eos_token_ids == (7,)
    minimal = {k: v for k, v in TINY_LLAMA.items()
               if k not in ("num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings")}
    _, d = config_from_dict(minimal)
    assert d.num_key_value_heads == 4 and d.head_dim == 16
    assert d.rms_norm_eps == 1e-5 and d.rope_theta == 10000.0 and d.tie_word_embeddings is False


def test_qwen3_differs_by_norm_and_eps_default():
    _, cfg = config_from_dict(TINY_QWEN3)
    assert cfg.qk_norm is True and cfg.q_width == 192 and cfg.q_width != cfg.hidden_size
    assert cfg.eos_token_ids == (3, 11)
    raw = dict(TINY_QWEN3)
    del raw["rms_norm_eps"]
    assert config_from_dict(raw)[1].rms_norm_eps == 1e-6


def test_round_trip(tmp_path):
    _, cfg = config_from_dict(TINY_QWEN3)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    _, again = load_config(str(tmp_path))
    assert again == cfg


def test_every_bad_key_is_named_at_once():
    raw = dict(TINY_LLAMA)
    del raw["vocab_size"]
    raw["hidden_size"] = -3
    raw["num_hidden_layers"] = "two"
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    text = str(err.value)
    assert "vocab_size" in text and "hidden_size" in text and "num_hidden_layers" in text


def test_heads_must_divide():
    raw = dict(TINY_LLAMA, num_attention_heads=4, num_key_value_heads=3)
    with pytest.raises(ConfigError, match="multiple"):
        config_from_dict(raw)
    raw = dict(TINY_LLAMA, hidden_size=66)
    del raw["head_dim"]
    with pytest.raises(ConfigError, match="head_dim"):
        config_from_dict(raw)


def test_unsupported_options_and_architectures():
    with pytest.raises(Unsupported, match="rope_scaling"):
        config_from_dict(dict(TINY_LLAMA, rope_scaling={"type": "linear", "factor": 2.0}))
    with pytest.raises(Unsupported, match="attention_bias"):
        config_from_dict(dict(TINY_LLAMA, attention_bias=True))
    with pytest.raises(Unsupported, match="supported: .*LlamaForCausalLM"):
        config_from_dict(dict(TINY_LLAMA, architectures=["MixtralForCausalLM"]))
    with pytest.raises(ConfigError):
        config_from_dict({"vocab_size": 3})
    with pytest.raises(ConfigError, match="no such file"):
        load_config("/nonexistent/folder")


def test_spec_names_every_size_from_the_config():
    arch, cfg = config_from_dict(TINY_QWEN3)
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 3 and [p.layer for p in spec.schedule] == [0, 1, 2]
    mixer = spec.layers[1].mixer
    assert mixer.kind == "attention" and mixer.params["n_heads"] == 6 and mixer.params["head_dim"] == 32
    assert mixer.params["position"]["params"] == {"rope_dim": 32, "base": 1000000.0, "scale": 1.0}
    assert spec.lm_head.weights["weight"] == "model.embed_tokens.weight"  # tied
    names = {e.name: e for e in spec.expected_tensors()}
    assert names["model.layers.2.self_attn.q_norm.weight"].shape == (32,)
    assert names["model.layers.0.mlp.down_proj.weight"].shape == (96, 160)
    assert "lm_head.weight" not in names
