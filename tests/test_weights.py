"""Safetensors files, loading by name with one error for everything, random weights (no GPU)."""
import json
import struct

import numpy as np
import pytest
import torch

import util
from air_b200.config import load_config
from air_b200.engine.engine import write_random_model
from air_b200.engine.model import Model
from air_b200.parts import registry
from air_b200.weights.loader import WeightError, load_tensors, random_tensors
from air_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


def specs_for(cfg):
    c = load_config(cfg)
    return Model(registry.architecture(c.architecture).build_spec(c)).tensor_specs()


def test_round_trip_and_plain_reader_agree(tmp_path):
    from plain import qwen2_plain as plain
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t)
    f = SafetensorsFile(path)
    assert sorted(f.names()) == ["a", "b", "c"]
    for k, v in t.items():
        assert torch.equal(f.tensor(k), v)
    p = plain.read_safetensors(path)
    assert np.array_equal(p["a"], t["a"].numpy()) and np.array_equal(p["b"], t["b"].float().numpy())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    write_random_model(str(tmp_path), util.TINY_A, 0, "bfloat16")
    specs = specs_for(util.TINY_A)
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(64, 65, dtype=torch.bfloat16)
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)   # the model is tied
    tensors["model.layers.7.extra"] = torch.zeros(2)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        load_tensors(str(tmp_path), specs, torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["lm_head.weight", "model.layers.7.extra"]
    assert err.wrong_shape == [("model.layers.0.self_attn.o_proj.weight", (64, 65), (64, 64))]
    for piece in ("missing (2)", "unexpected (2)", "wrong shape (1)", "file has [64, 65], model needs [64, 64]"):
        assert piece in str(err)


def test_absent_biases_are_allowed_as_in_air(tmp_path):
    write_random_model(str(tmp_path), util.TINY_A, 0, "bfloat16")
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names() if not n.endswith("proj.bias")}
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    got = load_tensors(str(tmp_path), specs_for(util.TINY_A), torch.bfloat16, "cpu")
    assert not any(n.endswith(".bias") for n in got)


def test_precision_rule_of_a_bfloat16_engine(tmp_path):
    """float32 engine: everything float32.  bfloat16 engine: a 32-bit tensor that its part computes with in 32
    bits (norm weights, biases) stays 32-bit; a 32-bit matrix is rounded to bfloat16 (to nearest even) and the
    load says so, unless the caller asks to keep it; float16 is rounded to bfloat16."""
    from air_b200.weights.loader import LoadReport
    write_random_model(str(tmp_path), util.TINY_A, 0, "bfloat16")
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del f
    wide = tensors["model.layers.0.mlp.down_proj.weight"].float() + 1e-4       # not representable in bfloat16
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    tensors["model.layers.0.self_attn.q_proj.bias"] = tensors["model.layers.0.self_attn.q_proj.bias"].float()
    tensors["model.layers.0.mlp.down_proj.weight"] = wide
    tensors["model.layers.1.mlp.down_proj.weight"] = tensors["model.layers.1.mlp.down_proj.weight"].to(torch.float16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    specs = specs_for(util.TINY_A)
    report = LoadReport()
    bf = load_tensors(str(tmp_path), specs, torch.bfloat16, "cpu", report=report)
    assert bf["model.norm.weight"].dtype == torch.float32                    # computed with in 32 bits: stays
    assert bf["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    assert bf["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert bf["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16  # a matrix: rounded, never a silent slow path
    assert torch.equal(bf["model.layers.0.mlp.down_proj.weight"], wide.to(torch.bfloat16))
    assert bf["model.layers.1.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert sorted(report.rounded) == ["model.layers.0.mlp.down_proj.weight", "model.layers.1.mlp.down_proj.weight"]
    assert sorted(report.kept_float32) == ["model.layers.0.self_attn.q_proj.bias", "model.norm.weight"]
    assert "rounded to bfloat16" in report.summary()
    kept = load_tensors(str(tmp_path), specs, torch.bfloat16, "cpu", keep_float32=True)
    assert kept["model.layers.0.mlp.down_proj.weight"].dtype == torch.float32
    assert torch.equal(kept["model.layers.0.mlp.down_proj.weight"], wide)
    fp = load_tensors(str(tmp_path), specs, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in fp.values())
    assert torch.equal(fp["model.embed_tokens.weight"], bf["model.embed_tokens.weight"].float())


def test_a_folder_of_shards_with_an_index(tmp_path):
    """model.safetensors.index.json maps every tensor to its shard, the form that large checkpoints have.  The
    load finds tensors by name whatever the files are (AIR: src/model/model.cpp:75-87); an index that puts a
    tensor in the wrong shard, or names a shard that is missing, is an error that says which."""
    folder = tmp_path / "m"
    write_random_model(str(folder), util.TINY_B, 1, "bfloat16")
    specs = specs_for(util.TINY_B)
    whole = load_tensors(str(folder), specs, torch.bfloat16, "cpu")
    f = SafetensorsFile(str(folder / "model.safetensors"))
    names = sorted(f.names())
    shards = {"model-00001-of-00002.safetensors": names[: len(names) // 2],
              "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for shard, members in shards.items():
        write_safetensors(str(folder / shard), {n: f.tensor(n).clone() for n in members})
    del f
    (folder / "model.safetensors").unlink()
    index = {"metadata": {}, "weight_map": {n: shard for shard, members in shards.items() for n in members}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    got = load_tensors(str(folder), specs, torch.bfloat16, "cpu")
    assert got.keys() == whole.keys() and all(torch.equal(got[k], whole[k]) for k in whole)
    # the index puts a tensor into the wrong shard
    wrong = dict(index["weight_map"])
    moved = shards["model-00001-of-00002.safetensors"][0]
    wrong[moved] = "model-00002-of-00002.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wrong}))
    with pytest.raises(SafetensorsError, match=f"'{moved}' is not in model-00002-of-00002.safetensors"):
        load_tensors(str(folder), specs, torch.bfloat16, "cpu")
    # a shard is missing
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    (folder / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(SafetensorsError, match="names the shard model-00002-of-00002.safetensors"):
        load_tensors(str(folder), specs, torch.bfloat16, "cpu")
    # a tensor that the index does not name: missing for the model, in ONE error with the rest
    write_safetensors(str(folder / "model-00002-of-00002.safetensors"),
                      {n: whole[n] for n in shards["model-00002-of-00002.safetensors"]})
    fewer = {k: v for k, v in index["weight_map"].items() if k != "model.norm.weight"}
    write_safetensors(str(folder / "model-00001-of-00002.safetensors"),
                      {n: whole[n] for n in shards["model-00001-of-00002.safetensors"] if n != "model.norm.weight"})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": fewer}))
    if "model.norm.weight" in shards["model-00002-of-00002.safetensors"]:
        write_safetensors(str(folder / "model-00002-of-00002.safetensors"),
                          {n: whole[n] for n in shards["model-00002-of-00002.safetensors"] if n != "model.norm.weight"})
    with pytest.raises(WeightError) as e:
        load_tensors(str(folder), specs, torch.bfloat16, "cpu")
    assert e.value.missing == ["model.norm.weight"]


def test_malformed_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    header = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)     # data shorter than the range
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    header = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                         "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="overlap"):
        SafetensorsFile(str(p))
    header = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError):
        load_tensors(str(tmp_path / "none"), [], torch.float32, "cpu")


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    specs = specs_for(util.TINY_B)
    a = random_tensors(specs, 1, torch.bfloat16)
    b = random_tensors(list(reversed(specs)), 1, torch.bfloat16)
    c = random_tensors(specs, 2, torch.bfloat16)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    w = a["model.layers.0.mlp.down_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.001
    n = a["model.layers.1.input_layernorm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.01
    write_random_model(str(tmp_path / "m"), util.TINY_B, 1, "bfloat16")
    cfg = json.loads((tmp_path / "m" / "config.json").read_text())
    assert cfg["architectures"] == ["Qwen2ForCausalLM"] and cfg["intermediate_size"] == 352
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    assert torch.equal(f.tensor("lm_head.weight"), a["lm_head.weight"])
