"""Typed configuration and the registry."""
import json

import pytest

from conftest import TINY_A, TINY_B


def test_qwen2_keys_and_defaults():
    from hfcpu_b200.config import config_from_dict
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert a.head_dim == 16                                  # default: hidden_size / heads (src/model.c:131)
    assert b.head_dim == 32 and b.vocab_size == 1000 and b.rope_theta == 1e6 and b.rms_norm_eps == 1e-5
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert [a.window_of_layer(l) for l in range(2)] == [0, 0]
    assert [b.window_of_layer(l) for l in range(3)] == [0, 64, 64]
    d = dict(TINY_A)
    del d["num_key_value_heads"], d["rms_norm_eps"], d["rope_theta"]
    c = config_from_dict(d)
    assert c.num_key_value_heads == 4 and c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0    # src/model.c:126-139


def test_round_trip_through_config_json(tmp_path):
    from hfcpu_b200.config import config_from_dict, load_config
    c = config_from_dict(TINY_B)
    c.save(str(tmp_path))
    assert load_config(str(tmp_path)) == c
    assert json.load(open(tmp_path / "config.json"))["architectures"] == ["Qwen2ForCausalLM"]


@pytest.mark.parametrize("change, error", [
    ({"num_hidden_layers": None}, "required key 'num_hidden_layers'"),
    ({"hidden_size": "64"}, "must be an integer"),
    ({"num_hidden_layers": 0}, "outside"),
    ({"num_key_value_heads": 3}, "unsupported attention geometry"),
    ({"head_dim": 15}, "odd"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"use_sliding_window": True, "sliding_window": 0}, "sliding_window"),
    ({"use_sliding_window": True, "sliding_window": 8, "max_window_layers": 5}, "max_window_layers"),
    ({"tie_word_embeddings": "yes"}, "true or false"),
    ({"eos_token_id": "x"}, "eos_token_id"),
])
def test_bad_configurations_are_refused(change, error):
    from hfcpu_b200.config import ConfigError, config_from_dict
    d = dict(TINY_A)
    d.update(change)
    if change.get("num_hidden_layers", 1) is None:
        del d["num_hidden_layers"]
    with pytest.raises(ConfigError, match=error):
        config_from_dict(d)


def test_registry():
    from hfcpu_b200.config import (ConfigError, UnsupportedError, config_from_dict, known_architectures,
                                   register_architecture, unregister_architecture)
    from hfcpu_b200.config import Qwen2Config
    assert {"Qwen2ForCausalLM", "qwen2"} <= set(known_architectures())
    d = dict(TINY_A, architectures=["LlamaForCausalLM"], model_type="llama")
    with pytest.raises(UnsupportedError, match="architecture 'LlamaForCausalLM' is not supported yet"):
        config_from_dict(d)
    d = dict(TINY_A)
    del d["architectures"]
    assert config_from_dict(d).architecture == "qwen2"        # model_type alone is enough
    del d["model_type"]
    with pytest.raises(ConfigError):
        config_from_dict(d)
    register_architecture("AliasForCausalLM", Qwen2Config)
    try:
        assert config_from_dict(dict(TINY_A, architectures=["AliasForCausalLM"])).hidden_size == 64
    finally:
        unregister_architecture("AliasForCausalLM")


def test_plan_is_data_and_is_checked():
    from hfcpu_b200.config import ConfigError, ScheduleEntry, config_from_dict
    import dataclasses
    plan = config_from_dict(TINY_B).plan()
    assert [e.layer for e in plan.schedule] == [0, 1, 2] and plan.layers[1].mixer.args["window"] == 64
    assert plan.layers[0].mixer.args["window"] == 0 and plan.head.args["tied_to"] is None
    bad = dataclasses.replace(plan, schedule=[ScheduleEntry(0), ScheduleEntry(7)])
    with pytest.raises(ConfigError):
        bad.validate()
    bad = dataclasses.replace(plan, schedule=[ScheduleEntry(0, cache_of=0)])
    with pytest.raises(ConfigError):
        bad.validate()
    ok = dataclasses.replace(plan, schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(2, cache_of=1)])
    ok.validate()
