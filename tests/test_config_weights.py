"""Configuration reading, the registry, safetensors I/O, the loader's one error, random weights."""
import os
import struct

import pytest
import torch

from tiny_configs import TINY_A, TINY_B, TINY_W

from nanoinfer_b200.config import ConfigError, EngineConfig, Qwen2Config, read_config_json
from nanoinfer_b200.registry import architecture_names, config_from_json_dict, plan_for
from nanoinfer_b200.weights import (SafetensorsError, WeightError, load_tensors, open_model_files,
                                    save_safetensors, write_random_model)


def test_config_reads_every_key():
    a, b = config_from_json_dict(TINY_A), config_from_json_dict(TINY_B)
    assert isinstance(a, Qwen2Config)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (b.intermediate_size, b.vocab_size, b.rope_theta, b.rms_norm_eps) == (320, 503, 1e6, 1e-5)
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.attention_bias and a.sliding_window == 0 and a.n_rep == 2 and b.n_rep == 6
    w = config_from_json_dict(TINY_W)
    assert w.sliding_window == 24 and w.max_window_layers == 1 and w.head_dim == 48


def test_config_defaults_and_variants():
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "num_key_value_heads", "rms_norm_eps",
                                                       "rope_theta", "max_position_embeddings")}
    c = config_from_json_dict(d)
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rms_norm_eps == 1e-6
    assert c.rope_theta == 10000.0 and c.max_position_embeddings == 4096
    d2 = dict(d, rope_parameters={"rope_type": "default", "rope_theta": 500000.0})
    assert config_from_json_dict(d2).rope_theta == 500000.0
    # a window value without the opt-in means full attention
    assert config_from_json_dict(dict(TINY_A, sliding_window=32768)).sliding_window == 0
    assert config_from_json_dict(dict(TINY_A, eos_token_id=[7, 9])).eos_token_id == 7
    assert config_from_json_dict(dict(TINY_A, attention_bias=False)).attention_bias is False


@pytest.mark.parametrize("patch,word", [
    ({"architectures": ["NoSuchModel"]}, "unknown architecture"),
    ({"architectures": []}, "architectures"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8}}, "rope_scaling"),
    ({"vocab_size": None}, "vocab_size"),
    ({"hidden_size": -4}, "hidden_size"),
    ({"num_hidden_layers": "two"}, "integer"),
    ({"head_dim": 15}, "even"),
])
def test_config_errors(patch, word):
    with pytest.raises(ConfigError) as e:
        config_from_json_dict(dict(TINY_A, **patch))
    assert word in str(e.value)


def test_registry_and_plan():
    assert "Qwen2ForCausalLM" in architecture_names()
    plan = plan_for(config_from_json_dict(TINY_B))
    names = [t.name for t in plan.tensor_specs()]
    assert "lm_head.weight" in names and "model.layers.2.self_attn.k_proj.bias" in names
    assert len(names) == 3 * 12 + 3
    plan_a = plan_for(config_from_json_dict(TINY_A))
    assert "lm_head.weight" not in [t.name for t in plan_a.tensor_specs()] and plan_a.ignored_tensors
    w = plan_for(config_from_json_dict(TINY_W))
    assert [l.parts["mixer"].params["window"] for l in w.layers] == [0, 24, 24]
    rt = config_from_json_dict(config_from_json_dict(TINY_W).to_json_dict())
    assert rt == config_from_json_dict(TINY_W)


def test_engine_config():
    assert EngineConfig(dtype="bf16", num_pages=4).dtype == "bfloat16"
    assert EngineConfig(dtype="fp32", max_cache_tokens=100, page_size=16).resolved_num_pages() == 7
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig().resolved_num_pages()


def test_safetensors_roundtrip_and_independent_reader(tmp_path):
    t = {"a.w": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(2, 2, 2), "d": torch.randn(4).half()}
    p = str(tmp_path / "model.safetensors")
    save_safetensors(p, t, {"k": "v"})
    f = open_model_files(str(tmp_path))[0]
    assert sorted(f.names()) == sorted(t) and f.metadata == {"k": "v"}
    for k, v in t.items():
        assert torch.equal(f.tensor(k), v) and f.tensor(k).dtype == v.dtype
    from safetensors import safe_open        # the published reader agrees with ours
    with safe_open(p, "pt") as g:
        for k, v in t.items():
            assert torch.equal(g.get_tensor(k), v)


def test_safetensors_damage(tmp_path):
    p = str(tmp_path / "model.safetensors")
    save_safetensors(p, {"x": torch.randn(8, 8)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-10])
    with pytest.raises(SafetensorsError, match="outside the file"):
        open_model_files(str(tmp_path))
    open(p, "wb").write(struct.pack("<Q", 10 ** 9) + raw[8:])
    with pytest.raises(SafetensorsError, match="header length"):
        open_model_files(str(tmp_path))
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        open_model_files(str(tmp_path))
    os.remove(p)
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        open_model_files(str(tmp_path))


def test_loader_reports_everything_at_once(tmp_path):
    cfg = config_from_json_dict(TINY_B)
    d = write_random_model(cfg, str(tmp_path / "m"), seed=1)
    plan = plan_for(cfg)
    good = load_tensors(d, plan)
    assert all(v.dtype == torch.bfloat16 for v in good.values())
    f = open_model_files(d)[0]
    t = {n: f.tensor(n) for n in f.names()}
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 10)
    t["model.extra.thing"] = torch.zeros(2)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_tensors(d, plan)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.extra.thing"]
    assert len(err.wrong_shape) == 1 and "q_proj.weight" in err.wrong_shape[0] and "[10, 10]" in err.wrong_shape[0]
    for word in ("missing", "unexpected", "wrong shapes", "model.norm.weight"):
        assert word in str(err)


def test_loader_keeps_dtypes_and_tolerates_a_stored_tied_head(tmp_path):
    cfg = config_from_json_dict(TINY_A)
    d = write_random_model(cfg, str(tmp_path / "m"), seed=2, dtype="float32")
    plan = plan_for(cfg)
    got = load_tensors(d, plan)
    assert all(v.dtype == torch.float32 for v in got.values())       # stored in 32-bit, stays so
    f = open_model_files(d)[0]
    t = {n: f.tensor(n) for n in f.names()}
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    t["model.norm.weight"] = t["model.norm.weight"].to(torch.bfloat16)
    t["model.layers.0.input_layernorm.weight"] = t["model.layers.0.input_layernorm.weight"].half()
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    got = load_tensors(d, plan)
    assert "lm_head.weight" not in got
    assert got["model.norm.weight"].dtype == torch.bfloat16
    # float16 -> float32: nothing is lost, whatever the engine's dtype is (bfloat16 would drop mantissa bits)
    assert got["model.layers.0.input_layernorm.weight"].dtype == torch.float32
    assert torch.equal(got["model.layers.0.input_layernorm.weight"],
                       t["model.layers.0.input_layernorm.weight"].float())


def test_loader_lists_wrong_element_types_with_the_other_faults(tmp_path):
    """A matrix, gain or bias stored as integers or booleans is an error of the checkpoint, listed in the
    one WeightError beside what is missing (nanoinfer/weights.py:56-68, cpp/src/serialize.cpp:18-64)."""
    cfg = config_from_json_dict(TINY_B)
    d = write_random_model(cfg, str(tmp_path / "m"), seed=1)
    plan = plan_for(cfg)
    f = open_model_files(d)[0]
    t = {n: f.tensor(n) for n in f.names()}
    t["model.layers.0.self_attn.k_proj.weight"] = t["model.layers.0.self_attn.k_proj.weight"].float().mul(100).to(torch.int8)
    t["model.layers.1.post_attention_layernorm.weight"] = torch.ones_like(
        t["model.layers.1.post_attention_layernorm.weight"], dtype=torch.bool)
    t["model.layers.2.self_attn.v_proj.bias"] = t["model.layers.2.self_attn.v_proj.bias"].to(torch.int32)
    del t["model.norm.weight"]
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_tensors(d, plan)
    err = e.value
    assert err.missing == ["model.norm.weight"]
    assert len(err.wrong_dtype) == 3
    joined = " ".join(err.wrong_dtype)
    for name, tag in (("k_proj.weight", "I8"), ("post_attention_layernorm.weight", "BOOL"), ("v_proj.bias", "I32")):
        assert name in joined and tag in joined
    assert "wrong element types (3)" in str(err) and "missing tensors (1)" in str(err)


def test_loader_wants_integers_for_an_integer_table(tmp_path):
    """A plan may declare an integer table (TensorSpec.integer): it is kept as int32, and floats in its place
    are refused."""
    import dataclasses
    cfg = config_from_json_dict(TINY_A)
    d = write_random_model(cfg, str(tmp_path / "m"), seed=3)
    plan = plan_for(cfg)
    from nanoinfer_b200.parts.spec import PartSpec, TensorSpec
    table = TensorSpec("toy.table", (5,), "bias", integer=True)
    plan2 = dataclasses.replace(plan, final_norm=PartSpec(plan.final_norm.kind, plan.final_norm.params,
                                                         {**plan.final_norm.tensors, "table": table}))
    f = open_model_files(d)[0]
    t = {n: f.tensor(n) for n in f.names()}
    t["toy.table"] = torch.arange(5, dtype=torch.int64)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    got = load_tensors(d, plan2)
    assert got["toy.table"].dtype == torch.int32 and got["toy.table"].tolist() == [0, 1, 2, 3, 4]
    t["toy.table"] = torch.arange(5, dtype=torch.float32)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_tensors(d, plan2)
    assert e.value.wrong_dtype and "integer table" in e.value.wrong_dtype[0]


def test_random_weights_are_reproducible_and_distributed_as_stated(tmp_path):
    cfg = config_from_json_dict(TINY_B)
    d1 = write_random_model(cfg, str(tmp_path / "m1"), seed=5, dtype="float32")
    d2 = write_random_model(cfg, str(tmp_path / "m2"), seed=5, dtype="float32")
    d3 = write_random_model(cfg, str(tmp_path / "m3"), seed=6, dtype="float32")
    assert read_config_json(d1) == read_config_json(d2)
    a, b, c = (open_model_files(d)[0] for d in (d1, d2, d3))
    for n in a.names():
        assert torch.equal(a.tensor(n), b.tensor(n))
    assert not torch.equal(a.tensor("lm_head.weight"), c.tensor("lm_head.weight"))
    w = a.tensor("model.embed_tokens.weight")
    assert abs(w.std().item() - 0.02) < 0.001 and abs(w.mean().item()) < 0.001
    g = a.tensor("model.layers.0.input_layernorm.weight")
    assert abs(g.mean().item() - 1.0) < 0.03 and abs(g.std().item() - 0.1) < 0.03
    assert abs(a.tensor("model.layers.0.self_attn.q_proj.bias").std().item() - 0.02) < 0.005
    assert config_from_json_dict(read_config_json(d1)) == cfg


def test_loader_reads_a_checkpoint_in_shards(tmp_path):
    """A folder with ``model.safetensors.index.json`` and several files gives the same tensors as one file;
    a tensor that no shard holds is reported with the others; a shard the index names but the folder
    lacks is an error that names the file."""
    import json
    from nanoinfer_b200.weights.safetensors_io import SafetensorsError
    cfg = config_from_json_dict(TINY_B)
    whole = write_random_model(cfg, str(tmp_path / "whole"), seed=4)
    plan = plan_for(cfg)
    want = load_tensors(whole, plan)
    f = open_model_files(whole)[0]
    names = sorted(f.names())
    parts = {"model-00001-of-00003.safetensors": names[0::3], "model-00002-of-00003.safetensors": names[1::3],
             "model-00003-of-00003.safetensors": names[2::3]}
    d = tmp_path / "sharded"
    d.mkdir()
    (d / "config.json").write_text((tmp_path / "whole" / "config.json").read_text())
    weight_map = {}
    for fn, ns in parts.items():
        save_safetensors(str(d / fn), {n: f.tensor(n) for n in ns})
        weight_map.update({n: fn for n in ns})
    (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    got = load_tensors(str(d), plan)
    assert set(got) == set(want) and all(torch.equal(got[n], want[n]) for n in want)
    # one tensor gone from its shard
    gone = parts["model-00002-of-00003.safetensors"][0]
    save_safetensors(str(d / "model-00002-of-00003.safetensors"),
                     {n: f.tensor(n) for n in parts["model-00002-of-00003.safetensors"][1:]})
    with pytest.raises(WeightError) as e:
        load_tensors(str(d), plan)
    assert e.value.missing == [gone] and not e.value.unexpected
    # a shard gone from the folder
    os.remove(d / "model-00003-of-00003.safetensors")
    with pytest.raises((SafetensorsError, OSError), match="model-00003-of-00003"):
        load_tensors(str(d), plan)
