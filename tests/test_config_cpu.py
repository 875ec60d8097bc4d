"""Configuration: typed reading of config.json, clear errors, the registries."""
import json

import pytest

import tiny
from kindi_b200.config import (ConfigError, SamplingParams, architecture, architectures, model_from_config,
                               model_from_dir, part_class, register_architecture, register_part)
from kindi_b200.config.spec import ScheduleEntry
from kindi_b200.models.nanbeige import LlamaConfig as ModelConfig


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
        model_from_dir(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        model_from_dir(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_C))
    cfg, spec = model_from_dir(str(tmp_path))
    assert cfg == ModelConfig.from_dict(tiny.TINY_C) and len(spec.layers) == 4


def test_unknown_keys_are_an_error_and_harmless_ones_are_not():
    """a key nothing reads is a model computed without it (the reference's rule for its own configuration,
    kindi/config.py:86-88); keys that carry no arithmetic pass"""
    ok = dict(tiny.TINY_A, transformers_version="4.55.0", use_cache=True, pad_token_id=0, initializer_range=0.02,
              pretraining_tp=1, attention_dropout=0.0, _name_or_path="x", max_position_embeddings=4096,
              rope_scaling=None, attention_bias=False, mlp_bias=False, hidden_act="silu", bos_token_id=1)
    assert ModelConfig.from_dict(ok).max_position_embeddings == 4096
    with pytest.raises(ConfigError) as e:
        ModelConfig.from_dict(dict(tiny.TINY_A, frobnicate=3, other_thing=True))
    assert "frobnicate" in str(e.value) and "other_thing" in str(e.value)
    # keys of related architectures that change the arithmetic: refused by name unless they say "off"
    for key, value in (("partial_rotary_factor", 0.5), ("attention_multiplier", 0.1), ("logits_scaling", 8.0),
                       ("residual_multiplier", 0.2), ("embedding_multiplier", 12.0), ("final_logit_softcapping", 30.0),
                       ("qk_norm", True), ("num_local_experts", 8), ("quantization_config", {"bits": 4}),
                       ("mlp_bias", True)):
        with pytest.raises(ConfigError) as e:
            ModelConfig.from_dict(dict(tiny.TINY_A, **{key: value}))
        assert key in str(e.value), key
    assert ModelConfig.from_dict(dict(tiny.TINY_A, partial_rotary_factor=1.0, logits_scaling=1.0, qk_norm=False))
    # a window that the folder says is not in use is not applied
    assert ModelConfig.from_dict(dict(tiny.TINY_A, sliding_window=16, use_sliding_window=False)).sliding_window is None


def test_another_architecture_reads_its_own_keys(tmp_path):
    """a folder of an architecture with other keys - no attention heads at all, a GELU feed-forward - loads through
    the registry: nothing of the Llama reader runs for it"""
    from kindi_b200.config import ConfigReader, LayerSpec, ModelSpec, PartSpec, default_schedule
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights import load_tensors
    from kindi_b200.weights.random_init import write_random_model

    def read(raw):
        r = ConfigReader(raw)
        r.ignore("architectures", "model_type")
        if r.string("hidden_act") != "gelu":
            raise ConfigError("config.json: the toy architecture is GELU only")
        out = dict(width=r.integer("d_model"), layers=r.integer("n_layer"), vocab=r.integer("vocab_size"),
                   inner=r.integer("d_inner"), eps=r.number("layer_norm_epsilon"), emb_scale=r.number("emb_scale", 1.0))
        r.finish()
        return out

    def build(c):
        norm = PartSpec("rmsnorm", {"eps": c["eps"]})
        block = PartSpec("prenorm", {"norm1": norm, "mixer": PartSpec("toy_cfg_mixer", {}), "norm2": norm,
                                     "feed_forward": PartSpec("toy_cfg_gelu", {"inner": c["inner"]})})
        return ModelSpec(architecture="ToyGeluLM", vocab_size=c["vocab"], width=c["width"],
                         layers=tuple(LayerSpec(block, "h.%d." % i) for i in range(c["layers"])),
                         schedule=default_schedule(c["layers"]), final_norm=norm, final_norm_prefix="ln_f.",
                         embedding=PartSpec("table", {"name": "wte", "vocab": c["vocab"], "scale": c["emb_scale"]}),
                         head=PartSpec("linear", {"name": "head", "tied_to": "wte", "vocab": c["vocab"],
                                                  "softcap": 30.0}))

    from kindi_b200.parts.base import FeedForward, Mixer

    class CfgMixer(Mixer):
        @classmethod
        def tensor_shapes(cls, spec, width):
            return {"mix.weight": (width, width), "mix.bias": (width,)}

        @classmethod
        def tensor_init(cls, spec, width):
            return {"mix.bias": "zero"}

    class CfgGelu(FeedForward):
        @classmethod
        def tensor_shapes(cls, spec, width):
            return {"fc.weight": (int(spec["inner"]), width), "proj.weight": (width, int(spec["inner"]))}

    register_part("mixer", "toy_cfg_mixer", CfgMixer, replace=True)
    register_part("feed_forward", "toy_cfg_gelu", CfgGelu, replace=True)
    register_architecture("ToyGeluLM", build, read, replace=True)
    raw = dict(architectures=["ToyGeluLM"], hidden_act="gelu", d_model=24, n_layer=2, vocab_size=50, d_inner=40,
               layer_norm_epsilon=1e-5, emb_scale=3.0, use_cache=True)
    cfg, spec = model_from_config(raw)
    assert cfg["width"] == 24 and spec.embedding["scale"] == 3.0 and spec.head["softcap"] == 30.0
    with pytest.raises(ConfigError) as e:
        model_from_config(dict(raw, num_attention_heads=4))           # not a key of this architecture
    assert "num_attention_heads" in str(e.value)
    d = write_random_model(str(tmp_path / "toy"), raw, seed=1, dtype="float32")
    shapes = expected_tensors(spec)
    assert set(shapes) == {"wte", "ln_f.weight"} | {"h.%d.%s" % (i, s) for i in range(2) for s in (
        "input_layernorm.weight", "self_attn.mix.weight", "self_attn.mix.bias", "post_attention_layernorm.weight",
        "mlp.fc.weight", "mlp.proj.weight")}
    assert tensor_inits(spec)["h.0.self_attn.mix.bias"] == "zero" and tensor_inits(spec)["ln_f.weight"] == "gain"
    t = load_tensors(d, shapes, run_dtype="float32", may_ignore=spec.may_ignore, copies=spec.copies)
    assert float(t["h.1.self_attn.mix.bias"].abs().sum()) == 0.0          # a bias is drawn as zero, not around one
    assert abs(float(t["h.0.input_layernorm.weight"].mean()) - 1.0) < 0.05  # a gain around one
    assert abs(float(t["h.0.self_attn.mix.weight"].mean())) < 0.01


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
    tied = architecture("llama").build_spec(ModelConfig.from_dict(tiny.TINY_B))
    assert tied.head["tied_to"] == tied.embedding["name"] == "model.embed_tokens.weight"
    assert model_from_config(tiny.TINY_A)[1].head["tied_to"] is None
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
