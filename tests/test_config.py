"""Configuration and registry: keys of config.json, defaults, refusals."""
import copy
import json

import pytest

from conftest import TINY_A, TINY_B, TINY_C
from imp_b200.config.engine_config import EngineConfig
from imp_b200.config.model_config import ConfigError, Qwen3Config
from imp_b200.config.registry import (config_from_dict, known_architectures, load_config, plan_for,
                                      register_architecture, unregister_architecture)


def test_reads_every_size_from_config_json():
    c = config_from_dict(TINY_B)
    assert isinstance(c, Qwen3Config)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size) == (3, 96, 6, 3, 32, 200, 503)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False
    assert [c.window_of_layer(i) for i in range(3)] == [0, 24, 24]


def test_defaults_head_dim_and_kv_heads():
    d = copy.deepcopy(TINY_A)
    del d["head_dim"], d["num_key_value_heads"]
    c = config_from_dict(d)
    assert c.head_dim == 16 and c.num_key_value_heads == 4


def test_layer_types_choose_window_per_layer():
    c = config_from_dict(TINY_C)
    assert [c.window_of_layer(i) for i in range(4)] == [9, 0, 9, 0]
    plan = plan_for(c)
    assert [l.mixer.params["window"] for l in plan.layers] == [9, 0, 9, 0]


def test_end_tokens_are_kept_as_a_list(tmp_path):
    assert config_from_dict(TINY_A).eos_token_ids == ()
    assert config_from_dict(dict(TINY_A, eos_token_id=9)).eos_token_ids == (9,)
    c = config_from_dict(dict(TINY_A, eos_token_id=[9, 200]))
    assert c.eos_token_ids == (9, 200)
    c.save(str(tmp_path))
    assert load_config(str(tmp_path)).eos_token_ids == (9, 200)


def test_round_trip_through_folder(tmp_path):
    c = config_from_dict(TINY_C)
    c.save(str(tmp_path))
    c2 = load_config(str(tmp_path))
    assert c2 == c
    assert json.load(open(tmp_path / "config.json"))["architectures"] == ["Qwen3ForCausalLM"]


@pytest.mark.parametrize("key", ["hidden_size", "num_attention_heads", "intermediate_size", "vocab_size",
                                 "num_hidden_layers", "rms_norm_eps"])
def test_missing_key_is_named(key):
    d = copy.deepcopy(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"attention_bias": True}, "attention_bias"),
    ({"head_dim": 24}, "multiple of 16"),
    ({"head_dim": 512}, "256"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"torch_dtype": "float16"}, "torch_dtype"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"vocab_size": 0}, "vocab_size"),
])
def test_refuses_what_it_cannot_run(patch, word):
    d = copy.deepcopy(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_unknown_architecture_lists_known():
    d = copy.deepcopy(TINY_A)
    d["architectures"] = ["NoSuchModel"]
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(d)
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in d.items() if k != "architectures"})


def test_registering_an_architecture():
    def plan(cfg):
        return plan_for(config_from_dict(TINY_A))
    register_architecture("MyToy", Qwen3Config, plan)
    try:
        assert "MyToy" in known_architectures()
        with pytest.raises(ValueError):
            register_architecture("MyToy", Qwen3Config, plan)
        d = copy.deepcopy(TINY_A)
        d["architectures"] = ["MyToy"]
        assert config_from_dict(d).architecture == "MyToy"
    finally:
        unregister_architecture("MyToy")


def test_plan_names_hf_tensors_and_ties_head():
    a = plan_for(config_from_dict(TINY_A)).expected_tensors()
    b = plan_for(config_from_dict(TINY_B)).expected_tensors()
    assert "lm_head.weight" not in a and "lm_head.weight" in b
    assert a["model.layers.1.self_attn.q_norm.weight"].shape == (16,)
    assert b["model.layers.2.self_attn.k_proj.weight"].shape == (3 * 32, 96)
    assert b["model.layers.0.mlp.down_proj.weight"].shape == (96, 200)
    assert len(a) == 1 + 2 * 11 + 1 and len(b) == 1 + 3 * 11 + 2


def test_missing_config_file(tmp_path):
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))


def test_engine_config_validation():
    EngineConfig().validate()
    with pytest.raises(ValueError):
        EngineConfig(compute_dtype="float16").validate()
    with pytest.raises(ValueError):
        EngineConfig(max_batch_size=64, max_batch_tokens=8).validate()
