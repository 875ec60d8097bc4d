"""Weights: reading safetensors by name, storage-type rules, the one error that lists everything, random folders."""
import json
import os
import struct

import pytest
import torch

import tiny
from kindi_b200.config import model_from_config
from kindi_b200.parts.model import expected_tensors
from kindi_b200.weights import WeightError, load_tensors, write_file
from kindi_b200.weights.random_init import write_random_model


def _expected(name):
    return expected_tensors(model_from_config(tiny.TINY[name][0])[1])


def test_random_folder_is_reproducible_and_readable_by_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file
    a = tiny.make_model(tmp_path / "a", "A")
    b = tiny.make_model(tmp_path / "b", "A")
    ta, tb = load_file(a + "/model.safetensors"), load_file(b + "/model.safetensors")
    assert set(ta) == set(_expected("A")) and all(torch.equal(ta[k], tb[k]) for k in ta)
    other = write_random_model(str(tmp_path / "c"), tiny.TINY_A, seed=5)
    tc = load_file(other + "/model.safetensors")
    assert not torch.equal(ta["model.embed_tokens.weight"], tc["model.embed_tokens.weight"])
    mine = load_tensors(a, _expected("A"))
    assert all(torch.equal(mine[k], ta[k]) for k in ta)
    assert "lm_head.weight" in ta and "lm_head.weight" not in _expected("B")          # B is tied
    w = ta["model.layers.0.mlp.down_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    assert abs(float(ta["model.norm.weight"].float().mean()) - 1.0) < 0.02


def test_storage_types(tmp_path):
    d = str(tmp_path)
    t = {"a": torch.randn(4, 3).to(torch.bfloat16), "b": torch.randn(5), "c": torch.randn(2, 2).to(torch.float16),
         "d": torch.arange(6, dtype=torch.int64).reshape(2, 3), "e": torch.randn(3, dtype=torch.float64)}
    write_file(os.path.join(d, "model.safetensors"), t)
    shapes = {k: tuple(v.shape) for k, v in t.items()}
    got = load_tensors(d, shapes, run_dtype="bfloat16")
    assert got["a"].dtype == torch.bfloat16 and torch.equal(got["a"], t["a"])
    assert got["b"].dtype == torch.float32 and torch.equal(got["b"], t["b"])         # 32-bit stays 32-bit
    assert got["c"].dtype == torch.float32 and torch.equal(got["c"], t["c"].float())
    assert got["d"].dtype == torch.int32 and got["d"].tolist() == t["d"].tolist()    # integer tables: int32
    assert got["e"].dtype == torch.float32
    got = load_tensors(d, shapes, run_dtype="float32")
    assert got["a"].dtype == torch.float32 and torch.equal(got["a"], t["a"].float())  # an exact widening


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from safetensors.torch import load_file
    src = tiny.make_model(tmp_path / "src", "A")
    t = load_file(src + "/model.safetensors")
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    d = str(tmp_path / "bad")
    os.makedirs(d)
    write_file(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_tensors(d, _expected("A"))
    err = e.value
    assert set(err.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert err.unexpected == ("model.layers.0.self_attn.q_proj.bias",)
    assert err.wrong_shape == ("model.layers.0.self_attn.k_proj.weight",)
    msg = str(err)
    for word in ("missing", "unexpected", "wrong shape", "model.norm.weight", "q_proj.bias", "[32, 64]", "[16, 64]"):
        assert word in msg


def test_untied_model_without_head_is_an_error(tmp_path):
    from safetensors.torch import load_file
    src = tiny.make_model(tmp_path / "src", "A")
    t = load_file(src + "/model.safetensors")
    del t["lm_head.weight"]
    d = str(tmp_path / "nohead")
    os.makedirs(d)
    write_file(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_tensors(d, _expected("A"))
    assert e.value.missing == ("lm_head.weight",)


def test_broken_files(tmp_path):
    d = str(tmp_path)
    with pytest.raises(WeightError):
        load_tensors(d, {"a": (1,)})                                   # no file at all
    p = os.path.join(d, "model.safetensors")
    write_file(p, {"a": torch.zeros(8, 8)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-40])                                     # truncated
    with pytest.raises(WeightError) as e:
        load_tensors(d, {"a": (8, 8)})
    assert "truncated" in str(e.value)
    open(p, "wb").write(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(WeightError):
        load_tensors(d, {"a": (8, 8)})
    open(p, "wb").write(b"abc")
    with pytest.raises(WeightError):
        load_tensors(d, {"a": (8, 8)})


def test_sharded_folder(tmp_path):
    d = str(tmp_path)
    write_file(os.path.join(d, "model-00001-of-00002.safetensors"), {"a": torch.ones(2, 2)})
    write_file(os.path.join(d, "model-00002-of-00002.safetensors"), {"b": torch.zeros(3)})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}, f)
    got = load_tensors(d, {"a": (2, 2), "b": (3,)})
    assert got["a"].sum() == 4 and got["b"].numel() == 3


def test_names_a_folder_may_hold_beside_what_the_model_reads(tmp_path):
    """a tied model that also stores its head is accepted when the head is the embedding table bit for bit and refused
    when it differs; rotary frequency buffers of older exports are ignored; anything else stays an error"""
    from safetensors.torch import load_file
    src = tiny.make_model(tmp_path / "src", "B")                       # B is tied
    spec = model_from_config(tiny.TINY_B)[1]
    t = load_file(src + "/model.safetensors")
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(16)
    d = str(tmp_path / "with_head")
    os.makedirs(d)
    write_file(os.path.join(d, "model.safetensors"), t)
    got = load_tensors(d, expected_tensors(spec), may_ignore=spec.may_ignore, copies=spec.copies)
    assert set(got) == set(expected_tensors(spec))
    with pytest.raises(WeightError):
        load_tensors(d, expected_tensors(spec))                        # without the architecture's say-so: unexpected
    t["lm_head.weight"][3, 5] += 1.0
    t["model.layers.0.self_attn.something_else"] = torch.ones(2)
    d2 = str(tmp_path / "other_head")
    os.makedirs(d2)
    write_file(os.path.join(d2, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_tensors(d2, expected_tensors(spec), may_ignore=spec.may_ignore, copies=spec.copies)
    assert "lm_head.weight != model.embed_tokens.weight" in str(e.value)
    assert "something_else" in str(e.value) and "inv_freq" not in str(e.value)


def test_wide_matrices_in_a_bfloat16_run_are_reported(tmp_path):
    src = tiny.make_model(tmp_path / "src", "A", "float32")
    said = []
    got = load_tensors(src, _expected("A"), run_dtype="bfloat16", log=said.append)
    assert got["model.layers.0.mlp.up_proj.weight"].dtype == torch.float32        # stored in 32-bit: stays so
    assert len(said) == 1 and "32-bit" in said[0] and "slower" in said[0]
    said.clear()
    load_tensors(tiny.make_model(tmp_path / "src", "A", "bfloat16"), _expected("A"), run_dtype="bfloat16", log=said.append)
    assert not said
