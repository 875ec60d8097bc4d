"""Configuration: typed reading of config.json, clear errors, the registries."""
import json
import os

import pytest

import tiny
from kindi_b200.config import (ConfigError, ModelConfig, SamplingParams, architecture, architectures, part_class,
                               register_architecture, register_part)
from kindi_b200.config.spec import ScheduleEntry


def test_reads_every_size_from_config():
    for name, (cfg, _) in tiny.TINY.items():
        c = ModelConfig.from_dict(cfg)
        assert c.vocab_size == cfg["vocab_size"] and c.hidden_size == cfg["hidden_size"]
        assert c.num_hidden_layers == cfg["num_hidden_layers"] and c.head_dim == cfg["head_dim"]
        assert c.rms_norm_eps == cfg["rms_norm_eps"] and c.rope_theta == cfg["rope_theta"]
        assert c.tie_word_embeddings == cfg.get("tie_word_embeddings", False)
        assert ModelConfig.from_dict(c.to_dict()) == c          # round trip


def test_defaults_follow_the_reference():
    d = dict(tiny.TINY_A)
    del d["head_dim"], d["rope_theta"]
    c = ModelConfig.from_dict(d)
    assert c.head_dim == d["hidden_size"] // d["num_attention_heads"]
    assert c.rope_theta == 10000.0
    d2 = dict(d, rope_parameters={"rope_theta": 123.0, "rope_type": "default"})
    assert ModelConfig.from_dict(d2).rope_theta == 123.0
    assert ModelConfig.from_dict(dict(tiny.TINY_B)).eos_token_ids == (5, 7)
    assert ModelConfig.from_dict(dict(tiny.TINY_A)).eos_token_ids == (2,)


@pytest.mark.parametrize("change,word", [
    ({"rms_norm_eps": None}, "rms_norm_eps"), ({"hidden_size": "64"}, "hidden_size"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"), ({"head_dim": 15}, "head_dim"),
    ({"attention_bias": True}, "attention_bias"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"), ({"vocab_size": 0}, "vocab_size"),
    ({"sliding_window": -1}, "sliding_window"), ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"architectures": None, "model_type": None}, "architectures"),
])
def test_errors_name_the_key(change, word):
    d = dict(tiny.TINY_A)
    d.update(change)
    with pytest.raises(ConfigError) as e:
        ModelConfig.from_dict(d)
    assert word in str(e.value)


def test_from_dir_errors(tmp_path):
    with pytest.raises(ConfigError):
        ModelConfig.from_dir(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        ModelConfig.from_dir(str(tmp_path))


def test_layer_windows():
    c = ModelConfig.from_dict(tiny.TINY_C)
    assert [c.layer_window(i) for i in range(4)] == [40, None, 40, None]
    d = dict(tiny.TINY_A, sliding_window=8)
    assert ModelConfig.from_dict(d).layer_window(1) == 8


def test_registry_names_and_spec():
    assert "LlamaForCausalLM" in architectures() and "NanbeigeForCausalLM" in architectures()
    with pytest.raises(KeyError) as e:
        architecture("NoSuchModel")
    assert "LlamaForCausalLM" in str(e.value)
    c = ModelConfig.from_dict(tiny.TINY_C)
    spec = architecture(c.architecture).build_spec(c)
    assert len(spec.layers) == 4 and [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    mix = [l.block["mixer"] for l in spec.layers]
    assert [m.get("window") for m in mix] == [40, None, 40, None]
    assert mix[0]["n_heads"] == 6 and mix[0]["n_kv_heads"] == 2 and mix[0]["head_dim"] == 48
    assert spec.layers[0].block["norm1"]["eps"] == 3e-6
    assert ModelConfig.from_dict(tiny.TINY_B).tie_word_embeddings
    assert architecture("llama").build_spec(ModelConfig.from_dict(tiny.TINY_B)).head_name is None
    with pytest.raises(KeyError):
        part_class("mixer", "no_such_mixer")
    with pytest.raises(KeyError):
        register_part("nonsense", "x", object)
    with pytest.raises(KeyError):
        register_architecture("LlamaForCausalLM", lambda c: None)


def test_schedule_validation():
    from dataclasses import replace
    c = ModelConfig.from_dict(tiny.TINY_A)
    spec = architecture(c.architecture).build_spec(c)
    bad = replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0)))
    with pytest.raises(ValueError):
        bad.validate()
    bad = replace(spec, schedule=(ScheduleEntry(0, 0, reads_cache_of=1), ScheduleEntry(1, 1)))
    with pytest.raises(ValueError):
        bad.validate()
    ok = replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
                                 ScheduleEntry(1, 3, reads_cache_of=1)))
    ok.validate()
    assert ok.n_cache_entries == 4


def test_sampling_params():
    p = SamplingParams()
    assert (p.temperature, p.top_p, p.top_k, p.min_p, p.repeat_penalty, p.repeat_last_n, p.max_tokens) == \
        (0.7, 0.8, 20, 0.0, 1.0, 64, 1024)                     # the reference's defaults (kindi/config.py:41-47)
    assert SamplingParams(temperature=0.0).greedy
    with pytest.raises(KeyError):
        SamplingParams.from_options(temperatur=1.0)
    with pytest.raises(ValueError):
        SamplingParams(order="other")
    assert SamplingParams.from_options(top_k=None, seed=3).seed == 3
