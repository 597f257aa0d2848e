"""Weight files: reading by name, one error for all that does not fit, random-weights mode (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

import xeno_rt_b200  # noqa: F401
from xeno_rt_b200.config import config_from_dict
from xeno_rt_b200.core import DType, WeightError
from xeno_rt_b200.weights import (check_tensors, load_weights, normal_values, read_safetensors,
                                  read_safetensors_header, tensor_key, write_random_model, write_safetensors)
from xeno_rt_b200.weights.loader import kept_dtype
from helpers import TINY_LLAMA, TINY_QWEN3


def _expected(raw):
    arch, cfg = config_from_dict(raw)
    return arch.build_spec(cfg).expected_tensors()


def test_safetensors_round_trip(tmp_path):
    tensors = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
               "b": torch.randn(5).to(torch.bfloat16), "c": torch.arange(4, dtype=torch.int32)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, metadata={"k": "v"})
    header, start = read_safetensors_header(path)
    assert start % 8 == 0 and header["b"]["dtype"] == "BF16" and header["a"]["shape"] == [2, 3]
    back = read_safetensors(path)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and torch.equal(back[k], tensors[k])


def test_random_model_folder_and_plain_reader_agree(tmp_path):
    from plain.files import read_model_folder
    folder = write_random_model(str(tmp_path / "m"), TINY_QWEN3, seed=1, dtype="bfloat16")
    cfg = json.load(open(os.path.join(folder, "config.json")))
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["torch_dtype"] == "bfloat16"
    _, plain = read_model_folder(folder)
    ours = read_safetensors(os.path.join(folder, "model.safetensors"))
    assert set(plain) == set(ours) == {e.name for e in _expected(TINY_QWEN3)}
    for k in ours:
        assert ours[k].dtype == torch.bfloat16
        assert np.array_equal(ours[k].float().numpy(), plain[k])
    w = plain["model.layers.0.mlp.gate_proj.weight"]
    assert abs(w.std() - 0.02) < 0.002 and abs(w.mean()) < 0.002
    n = plain["model.layers.1.input_layernorm.weight"]
    assert abs(n.mean() - 1.0) < 0.05 and 0.05 < n.std() < 0.15


def test_generator_is_counter_based_and_seeded():
    key = tensor_key(5, "some.tensor")
    whole = normal_values(key, 100, 0.0, 1.0)
    assert np.array_equal(whole[40:60], normal_values(key, 20, 0.0, 1.0, start=40))
    assert not np.array_equal(whole, normal_values(tensor_key(6, "some.tensor"), 100, 0.0, 1.0))
    assert not np.array_equal(whole, normal_values(tensor_key(5, "other.tensor"), 100, 0.0, 1.0))
    big = normal_values(key, 200000, 0.0, 1.0)
    assert abs(big.mean()) < 0.01 and abs(big.std() - 1.0) < 0.01


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_LLAMA, seed=0, dtype="float32")
    path = os.path.join(folder, "model.safetensors")
    tensors = read_safetensors(path)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)  # ignorable
    write_safetensors(path, tensors)
    with pytest.raises(WeightError) as err:
        load_weights(folder, _expected(TINY_LLAMA), DType.F32, "cpu", ignorable=("*.rotary_emb.inv_freq",))
    text = str(err.value)
    assert "missing tensors (2)" in text and "model.layers.1.mlp.up_proj.weight" in text and "model.norm.weight" in text
    assert "unexpected tensors (1)" in text and "q_proj.bias" in text and "inv_freq" not in text
    assert "wrong shape or dtype (1)" in text and "shape [16, 64], expected [32, 64]" in text


def test_tied_model_rejects_a_separate_output_matrix(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_QWEN3, seed=1, dtype="bfloat16")
    path = os.path.join(folder, "model.safetensors")
    tensors = read_safetensors(path)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(path, tensors)
    with pytest.raises(WeightError, match="unexpected tensors.*lm_head.weight"):
        load_weights(folder, _expected(TINY_QWEN3), DType.BF16, "cpu")


def test_kept_dtypes(tmp_path):
    assert kept_dtype("matrix", torch.float32, DType.BF16) == torch.bfloat16
    assert kept_dtype("vector", torch.float32, DType.BF16) == torch.float32  # stored in 32-bit, stays so
    assert kept_dtype("vector", torch.bfloat16, DType.BF16) == torch.bfloat16
    assert kept_dtype("matrix", torch.bfloat16, DType.F32) == torch.float32
    assert kept_dtype("int", torch.int64, DType.BF16) == torch.int32
    folder = write_random_model(str(tmp_path / "m"), TINY_LLAMA, seed=0, dtype="float32")
    loaded = load_weights(folder, _expected(TINY_LLAMA), DType.BF16, "cpu")
    assert loaded["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert loaded["model.norm.weight"].dtype == torch.float32


def test_broken_files(tmp_path):
    with pytest.raises(WeightError, match="no such file"):
        read_safetensors_header(str(tmp_path / "none.safetensors"))
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(WeightError, match="shorter"):
        read_safetensors_header(str(p))
    p = tmp_path / "long.safetensors"
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightError, match="header length"):
        read_safetensors_header(str(p))


def test_check_tensors_passes_when_all_fits():
    exp = _expected(TINY_LLAMA)
    header = {e.name: {"dtype": "F32", "shape": list(e.shape)} for e in exp}
    check_tensors(exp, header)


def _load(folder, raw, dtype=DType.F32, **kw):
    arch, cfg = config_from_dict(raw)
    spec = arch.build_spec(cfg)
    return load_weights(folder, spec.expected_tensors(), dtype, "cpu", spec.ignorable_tensors, **kw), spec


def test_a_sharded_folder_loads_to_the_same_tensors_as_the_single_file(tmp_path):
    """Three shards and their index against the one-file folder of the same seed: every tensor
    bit for bit, also the tensors that land side by side in one shared buffer."""
    one = write_random_model(str(tmp_path / "one"), TINY_QWEN3, seed=1, dtype="bfloat16")
    three = write_random_model(str(tmp_path / "three"), TINY_QWEN3, seed=1, dtype="bfloat16", shards=3)
    files = sorted(f for f in os.listdir(three) if f.endswith(".safetensors"))
    assert files == [f"model-0000{i}-of-00003.safetensors" for i in (1, 2, 3)]
    assert not os.path.exists(os.path.join(three, "model.safetensors"))
    index = json.load(open(os.path.join(three, "model.safetensors.index.json")))
    assert set(index["weight_map"].values()) == set(files)
    stats = {}
    a, spec = _load(one, TINY_QWEN3, DType.BF16)
    b, _ = _load(three, TINY_QWEN3, DType.BF16, fused_groups=spec.fused_groups(), stats=stats)
    assert set(a) == set(b) and stats["files"] == 3
    for name in a:
        assert a[name].dtype == b[name].dtype and torch.equal(a[name], b[name]), name
    group = ("model.layers.1.self_attn.q_proj.weight", "model.layers.1.self_attn.k_proj.weight",
             "model.layers.1.self_attn.v_proj.weight")
    assert group in spec.fused_groups()
    fused = b.fused[group]
    assert torch.equal(fused, torch.cat([a[n] for n in group]))
    assert b[group[1]].data_ptr() == fused[192:].data_ptr()  # a view of the shared buffer: no second copy


def test_loading_holds_no_more_of_the_file_than_a_staging_piece(tmp_path, monkeypatch):
    """Tensors go to the device in pieces through a staging buffer of fixed size: with the piece set
    to 1 KiB a folder of 300 KB loads with 1 KiB in flight at any time, bit for bit."""
    from xeno_rt_b200.weights import loader
    folder = write_random_model(str(tmp_path / "m"), TINY_QWEN3, seed=4, dtype="float32", shards=2)
    whole, _ = _load(folder, TINY_QWEN3)
    monkeypatch.setattr(loader, "STAGING_BYTES", 1024)
    stats = {}
    pieces, _ = _load(folder, TINY_QWEN3, stats=stats)
    assert 0 < stats["peak_staging_bytes"] <= 1024
    largest = max(t.numel() * t.element_size() for t in whole.values())
    assert largest > 50 * 1024
    for name in whole:
        assert torch.equal(whole[name], pieces[name])


def test_one_error_for_a_broken_sharded_folder(tmp_path):
    """A shard that is gone, a tensor that the index sends to the wrong shard, a tensor held by two
    shards, a tensor no shard holds and a wrong shape: all in ONE error."""
    from xeno_rt_b200.weights import locate_tensors
    folder = write_random_model(str(tmp_path / "m"), TINY_LLAMA, seed=0, dtype="float32", shards=3)
    index_path = os.path.join(folder, "model.safetensors.index.json")
    index = json.load(open(index_path))
    files = sorted(set(index["weight_map"].values()))
    first = read_safetensors(os.path.join(folder, files[0]))
    second = read_safetensors(os.path.join(folder, files[1]))
    moved = sorted(second)[0]
    dup = sorted(first)[0]
    second[dup] = first[dup].clone()                       # held by two shards
    wrong = sorted(second)[-1]
    second[wrong] = torch.zeros(3, 3)                       # wrong shape
    write_safetensors(os.path.join(folder, files[1]), second)
    index["weight_map"][moved] = files[0]                  # the index points at a shard that does not hold it
    index["weight_map"]["model.phantom.weight"] = files[2]  # shard 3 is deleted below
    json.dump(index, open(index_path, "w"))
    os.remove(os.path.join(folder, files[2]))
    with pytest.raises(WeightError) as err:
        _load(folder, TINY_LLAMA)
    text = str(err.value)
    assert text.count("does not fit the model") == 1
    assert f"missing shard file: {files[2]}" in text
    assert "listed in the index but absent from their shard" in text and moved in text
    assert "held by two shards (1)" in text and dup in text
    assert "missing tensors" in text  # those of the deleted shard
    assert "wrong shape or dtype" in text and f"{wrong}: shape [3, 3]" in text
    header, where, problems, source = locate_tensors(folder)
    assert source.endswith("index.json") and len(problems) >= 3
    # an index that is not an index
    open(index_path, "w").write("{\"weight_map\": 3}")
    with pytest.raises(WeightError, match="weight_map"):
        _load(folder, TINY_LLAMA)
