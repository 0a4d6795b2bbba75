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


def test_precision_kept_as_stored(tmp_path):
    write_random_model(str(tmp_path), util.TINY_A, 0, "bfloat16")
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    specs = specs_for(util.TINY_A)
    bf = load_tensors(str(tmp_path), specs, torch.bfloat16, "cpu")
    assert bf["model.norm.weight"].dtype == torch.float32          # stored in 32 bits: stays
    assert bf["model.embed_tokens.weight"].dtype == torch.bfloat16
    fp = load_tensors(str(tmp_path), specs, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in fp.values())
    assert torch.equal(fp["model.embed_tokens.weight"], bf["model.embed_tokens.weight"].float())


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
