"""Configuration and registry (no GPU)."""
import json

import pytest

import util
from air_b200.config import ConfigError, Qwen2Config, load_config
from air_b200.parts import registry
from air_b200.engine.model import Model


def test_reads_every_size_from_config_json():
    for cfg, _ in util.CONFIGS.values():
        c = load_config(cfg)
        assert isinstance(c, Qwen2Config)
        assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (
            cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"])
        assert c.head_dim == cfg["hidden_size"] // cfg["num_attention_heads"]
        assert c.rope_theta == cfg["rope_theta"] and c.rms_norm_eps == cfg["rms_norm_eps"]
        assert load_config(c.to_dict()) == c


def test_kv_heads_default_to_heads():
    cfg = dict(util.TINY_A)
    del cfg["num_key_value_heads"]
    assert load_config(cfg).num_key_value_heads == cfg["num_attention_heads"]


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads", "intermediate_size",
                                 "vocab_size", "max_position_embeddings", "rope_theta", "rms_norm_eps"])
def test_missing_key_is_a_data_error(key):
    cfg = dict(util.TINY_A)
    del cfg[key]
    with pytest.raises(ConfigError) as e:
        load_config(cfg)
    assert e.value.kind == "data_error" and key in str(e.value)


@pytest.mark.parametrize("change, kind", [
    ({"hidden_size": 66}, "data_error"), ({"num_key_value_heads": 3}, "data_error"),
    ({"rms_norm_eps": 0.0}, "data_error"), ({"rope_theta": -1.0}, "data_error"),
    ({"num_hidden_layers": 0}, "data_error"), ({"num_hidden_layers": "2"}, "data_error"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "unsupported"), ({"hidden_act": "gelu"}, "unsupported"),
    ({"head_dim": 32}, "unsupported"), ({"model_type": "llama"}, "unsupported"),
    ({"use_sliding_window": True, "sliding_window": None}, "data_error"), ({"eos_token_id": 999}, "data_error"),
])
def test_refusals(change, kind):
    with pytest.raises(ConfigError) as e:
        load_config(dict(util.TINY_A, **change))
    assert e.value.kind == kind


def test_unknown_architecture_is_unsupported():
    with pytest.raises(ConfigError) as e:
        load_config(dict(util.TINY_A, architectures=["LlamaForCausalLM"]))
    assert e.value.kind == "unsupported" and "Qwen2ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        load_config({"hidden_size": 8})


def test_window_field_without_the_switch_is_ignored():
    c = load_config(util.TINY_B)
    assert c.sliding_window == 4096 and all(c.layer_window(i) is None for i in range(3))
    w = load_config(util.TINY_W)
    assert [w.layer_window(i) for i in range(3)] == [None, 40, 40]


def test_spec_chooses_parts_layer_by_layer():
    w = load_config(util.TINY_W)
    spec = registry.architecture(w.architecture).build_spec(w)
    assert [b.part("mixer")["window"] for b in spec.layers] == [None, 40, 40]
    assert [r.layer for r in spec.order] == [0, 1, 2] and spec.output_name == "lm_head.weight"
    model = Model(spec)
    needs = model.cache_needs()
    assert needs[0] != needs[1] and needs[1] == needs[2]
    names = {s.name for s in model.tensor_specs()}
    assert "model.layers.2.self_attn.k_proj.bias" in names and "model.norm.weight" in names
    tied = load_config(util.TINY_A)
    assert registry.architecture(tied.architecture).build_spec(tied).output_name is None


def test_config_json_file(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(util.TINY_B))
    assert load_config(str(tmp_path)).vocab_size == util.TINY_B["vocab_size"]
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nothing"))
