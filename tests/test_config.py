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


def test_options_that_would_be_ignored_are_refused():
    with pytest.raises(Unsupported, match="hidden_act"):
        config_from_dict(dict(TINY_LLAMA, hidden_act="gelu"))
    with pytest.raises(Unsupported, match="partial_rotary_factor"):
        config_from_dict(dict(TINY_QWEN3, partial_rotary_factor=0.5))
    with pytest.raises(Unsupported, match="mlp_bias"):
        config_from_dict(dict(TINY_LLAMA, mlp_bias=True))
    with pytest.raises(Unsupported, match="use_sliding_window"):
        config_from_dict(dict(TINY_QWEN3, use_sliding_window=True))
    config_from_dict(dict(TINY_LLAMA, hidden_act="silu", partial_rotary_factor=1.0, mlp_bias=False))


def test_stop_ids_of_generation_config_join_those_of_config(tmp_path):
    """Folders of chat models list the ids that end a turn in generation_config.json."""
    (tmp_path / "config.json").write_text(json.dumps(TINY_LLAMA))          # eos_token_id 7
    assert load_config(str(tmp_path))[1].eos_token_ids == (7,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [9, 7, 12], "temperature": 0.6}))
    arch, cfg = load_config(str(tmp_path))
    assert cfg.eos_token_ids == (7, 9, 12)
    assert arch.build_spec(cfg).stop_ids == (7, 9, 12)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 5}))
    assert load_config(str(tmp_path))[1].eos_token_ids == (7, 5)
    raw = {k: v for k, v in TINY_LLAMA.items() if k != "eos_token_id"}
    (tmp_path / "config.json").write_text(json.dumps(raw))
    assert load_config(str(tmp_path))[1].eos_token_ids == (5,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": "end"}))
    with pytest.raises(ConfigError, match="generation_config.json.*eos_token_id"):
        load_config(str(tmp_path))
    (tmp_path / "generation_config.json").write_text("{")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))


def test_spec_names_every_size_from_the_config():
    arch, cfg = config_from_dict(TINY_QWEN3)
    spec = arch.build_spec(cfg)
    assert len(spec.layers) == 3 and [p.layer for p in spec.schedule] == [0, 1, 2]
    mixer = spec.layers[1].parts["mixer"][1]
    assert mixer.kind == "attention" and mixer.params["n_heads"] == 6 and mixer.params["head_dim"] == 32
    assert mixer.params["position"]["params"] == {"rope_dim": 32, "base": 1000000.0, "scale": 1.0}
    assert spec.lm_head.weights["weight"] == "model.embed_tokens.weight"  # tied
    names = {e.name: e for e in spec.expected_tensors()}
    assert names["model.layers.2.self_attn.q_norm.weight"].shape == (32,)
    assert names["model.layers.0.mlp.down_proj.weight"].shape == (96, 160)
    assert "lm_head.weight" not in names


def test_which_kernel_takes_a_decode_product_of_few_rows():
    """The choice between the two weight-streaming kernels is host arithmetic over the product's sizes
    (here for a device of 148 multiprocessors): the tcgen05 kernel where its tiles of 128 weight rows,
    times its splits of K, fill the multiprocessors; the cp.async kernel else, and for products that add
    into the residual stream up to 8 rows, and beyond below K = 8,192, unless its own rounds of blocks fill badly."""
    from xeno_rt_b200.core import KernelError
    from xeno_rt_b200.csrc import ops
    from xeno_rt_b200.parts.linear_bf16 import tcgen05_for_few_rows as choice
    try:
        ops.library()  # the arithmetic lives beside the kernel it describes; building needs nvcc, not a GPU
    except KernelError as exc:
        pytest.skip(f"the kernel library cannot be built here: {exc}")
    sms = 148
    for rows in (1, 8, 16):
        # width 4,096, inner 14,336, vocabulary 128,256, 32 + 2 x 8 heads of 128
        assert not choice(sms, rows, 6144, 4096, "store")      # 48 tiles x 3 splits, more than the device's 45 clusters of 3
        assert choice(sms, rows, 5120, 4096, "store")          # 40 tiles x 3 splits as clusters
        assert choice(sms, rows, 14336, 4096, "swiglu")        # 112 items
        assert choice(sms, rows, 128256, 4096, "store")        # 1,002 tiles: seven rounds, 0.97 full
        assert not choice(sms, rows, 4096, 4096, "accumulate")
        assert choice(sms, rows, 4096, 14336, "accumulate") == (rows > 8)  # K >= 8,192: from 9 rows on
        # width 5,120, inner 25,600, 64 + 2 x 8 heads of 128
        assert not choice(sms, rows, 10240, 5120, "store")     # 80 items: 0.54 full
        assert not choice(sms, rows, 25600, 5120, "swiglu")    # 200 tiles: two rounds, 0.68 full
        assert choice(sms, rows, 5120, 25600, "accumulate") == (rows > 8)
        assert choice(sms, rows, 5120, 8192, "accumulate") == (rows > 8)  # 320 blocks of 16 rows: one round


def test_decode_attention_splits_cover_the_context_and_fill_the_rounds():
    """How decode attention cuts a context into splits is host arithmetic: every key belongs to one split,
    splits are whole cache blocks, and the counts are the ones that were measured fastest at 4,096 keys
    and 8 kv heads (few sequences: many splits that merge inside a cluster of at most 16 blocks; many
    sequences: few splits that fill the last round of blocks)."""
    from xeno_rt_b200.parts.attention_bf16 import CLUSTER_MAX_SPLITS, decode_split
    for n_seqs in (1, 2, 3, 8, 17, 64, 300):
        for kv_heads in (1, 2, 8):
            for context in (1, 63, 64, 65, 200, 4096, 5000, 32768):
                chunk, splits = decode_split(n_seqs, kv_heads, context, 148)
                blocks = (context + 63) // 64
                assert chunk % 64 == 0 and splits >= 1
                assert chunk * splits >= context                 # every key is in a split
                assert chunk * (splits - 1) < blocks * 64        # and no split is empty
    assert [decode_split(b, 8, 4096, 148)[1] for b in (1, 2, 4, 8, 16, 32, 64)] == [16, 16, 8, 4, 2, 3, 4]
    assert decode_split(1, 8, 32768, 148)[1] <= CLUSTER_MAX_SPLITS
    # unequal lengths: what a sequence holds on average decides how many blocks have work, so the keys are cut
    # finer when most sequences are far shorter than the longest; a mean as long as the longest changes nothing
    for n_seqs in (8, 16, 64):
        assert decode_split(n_seqs, 8, 4096, 148, 4096) == decode_split(n_seqs, 8, 4096, 148)
        assert decode_split(n_seqs, 8, 4096, 148, 1024)[1] > decode_split(n_seqs, 8, 4096, 148)[1]
        for mean in (1, 300, 1024, 5000):
            chunk, splits = decode_split(n_seqs, 8, 4096, 148, mean)
            assert chunk % 64 == 0 and chunk * splits >= 4096 and chunk * (splits - 1) < 4096
    # a windowed layer: the kernels count its splits from the cache block of the first visible key, so the keys to
    # cut are the window and what is left of that block, however long the sequence is
    from xeno_rt_b200.parts.attention_bf16 import visible_span
    assert visible_span(4096, 0) == 4096 and visible_span(40, 100) == 40
    for window in (1, 2, 63, 64, 65, 100, 128, 1000):
        span = visible_span(1 << 20, window)
        assert span % 64 == 0
        for length in range(1, 400):  # the newest key is length - 1; the first visible one max(0, length - window)
            first_block_key = max(0, length - window) // 64 * 64
            assert length - first_block_key <= span
        assert span - 64 < window + 63  # and not a block more than the worst case needs


def test_the_merging_block_of_decode_attention_is_never_given_more_splits_than_its_shared_memory_holds():
    """The block that merges a (token, kv head)'s splits inside the attention kernel keeps
    group * (2 * splits + 1) floats in its dynamic shared memory.  For every head-size class and group
    the launcher's limit fits the smallest launch (12 KB at head size 16), and the engine's own split
    counts (at most 64) stay under it wherever the merge is fused."""
    from xeno_rt_b200.csrc import ops
    for head_dim in range(16, 257, 16):
        cp = max(4 * 64 * (head_dim * 2 + 16), 8 * 16 * (2 + head_dim + 8) * 4)
        for group in (1, 2, 4, 5, 8, 16):
            limit = ops.attention_decode_fused_max_splits(head_dim, group)
            smallest = min(cp, 4 * (head_dim // 64) * 8192) if head_dim % 64 == 0 else cp  # the TMA tiles
            assert limit >= 1 and group * (2 * limit + 1) * 4 <= smallest
    assert ops.attention_decode_fused_max_splits(16, 16) < 96      # the advised overflow case is now refused
    assert ops.attention_decode_fused_max_splits(64, 16) < 288
    assert ops.attention_decode_fused_max_splits(128, 4) >= 64     # the engine's cases are all fused
    with pytest.raises(Exception):
        ops.attention_decode_fused_max_splits(20, 4)
