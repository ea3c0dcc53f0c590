"""Configuration and registry: what is accepted, what is refused, what the defaults are.

The accept / reject table mirrors the reference's own tests in meaning
(src/models/qwen3/config.rs:228-323, src/models/registry.rs:54-64).
"""
import copy

import pytest

from llm_infer_rust_b200 import (Architecture, ConfigError, Qwen3Config, register_architecture,
                                 registered_architectures, resolve_architecture)


def raw():
    return {"model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"], "hidden_size": 16,
            "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
            "intermediate_size": 32, "vocab_size": 64, "max_position_embeddings": 128,
            "rope_theta": 1000000.0, "rms_norm_eps": 0.00001, "tie_word_embeddings": True}


def test_sizes_come_from_the_keys():
    c = Qwen3Config.parse(raw())
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (16, 2, 4, 2)
    assert c.head_dim == 4 and c.intermediate_size == 32 and c.vocab_size == 64
    assert c.rope_theta == 1000000.0 and c.rms_norm_eps == 0.00001 and c.tie_word_embeddings is True
    r = raw()
    r["head_dim"] = 8                      # attention width independent of hidden_size
    assert Qwen3Config.parse(r).head_dim == 8


@pytest.mark.parametrize("field,value", [
    ("rope_scaling", {"rope_type": "linear", "factor": 2.0}), ("rope_parameters", {}),
    ("quantization_config", {}), ("compression_config", {}), ("attention_bias", True), ("mlp_bias", True),
    ("use_sliding_window", True),          # without a sliding_window length
    ("use_sliding_window", "yes"), ("hidden_act", "gelu"), ("qk_norm", False),
    ("layer_types", ["full_attention", "sliding_attention"]),   # asks for a window that is switched off
    ("layer_types", ["full_attention"]), ("layer_types", ["full_attention", "linear_attention"]),
    ("rms_norm_eps", 0.0), ("rope_theta", -1.0), ("rope_theta", float("inf")),
    ("tie_word_embeddings", "true"), ("tie_word_embeddings", None),
    ("num_hidden_layers", 0), ("num_hidden_layers", 2.5), ("num_hidden_layers", True),
    ("num_key_value_heads", 3), ("head_dim", 3), ("vocab_size", -4),
    ("max_position_embeddings", None), ("max_position_embeddings", "invalid"),
    ("rope_theta", None), ("rope_theta", "invalid"), ("rms_norm_eps", None), ("torch_dtype", "int8"),
    ("eos_token_id", 64), ("eos_token_id", [1, -1]),
])
def test_refused(field, value):
    r = raw()
    r[field] = value
    with pytest.raises(ConfigError):
        Qwen3Config.parse(r)


@pytest.mark.parametrize("field", ["hidden_size", "num_hidden_layers", "num_attention_heads",
                                   "intermediate_size", "vocab_size"])
def test_required(field):
    r = raw()
    del r[field]
    with pytest.raises(ConfigError, match=field):
        Qwen3Config.parse(r)


def test_metadata_and_a_dormant_window_are_permitted():
    r = raw()
    r.update(transformers_version="metadata", use_sliding_window=False, sliding_window=4096,
             layer_types=["full_attention", "full_attention"], rope_scaling=None, max_window_layers=1)
    c = Qwen3Config.parse(r)
    assert c.layer_windows == (None, None)


def test_head_dim_needs_exact_division_when_omitted():
    r = raw()
    r["hidden_size"] = 17
    with pytest.raises(ConfigError):
        Qwen3Config.parse(r)
    r["head_dim"] = 4
    assert Qwen3Config.parse(r).head_dim == 4


def test_defaults():
    r = raw()
    for f in ("max_position_embeddings", "rope_theta", "rms_norm_eps", "tie_word_embeddings",
              "num_key_value_heads"):
        del r[f]
    c = Qwen3Config.parse(r)
    assert c.max_position_embeddings == 8192 and c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6
    assert c.tie_word_embeddings is False and c.num_key_value_heads == 4 and c.head_dim == 4
    assert c.checkpoint_dtype == "float32" and c.eos_token_ids == ()


def test_eos_forms():
    r = raw()
    r["eos_token_id"] = 7
    assert Qwen3Config.parse(r).eos_token_ids == (7,)
    r["eos_token_id"] = [7, 9]
    assert Qwen3Config.parse(r).eos_token_ids == (7, 9)
    r["eos_token_id"] = []
    assert Qwen3Config.parse(r).eos_token_ids == ()


def test_window_by_layer_types_and_by_max_window_layers():
    r = raw()
    r.update(use_sliding_window=True, sliding_window=8, layer_types=["sliding_attention", "full_attention"])
    assert Qwen3Config.parse(r).layer_windows == (8, None)
    del r["layer_types"]
    r["max_window_layers"] = 1
    assert Qwen3Config.parse(r).layer_windows == (None, 8)


def test_model_spec_is_data_chosen_layer_by_layer():
    r = raw()
    r.update(use_sliding_window=True, sliding_window=8, layer_types=["sliding_attention", "full_attention"])
    spec = Qwen3Config.parse(r).model_spec()
    assert [e.layer for e in spec.run_list] == [0, 1] and all(e.reads is None for e in spec.run_list)
    assert spec.layers[0]["mixer"]["window"] == 8 and spec.layers[1]["mixer"]["window"] is None
    assert spec.layers[0]["mixer"]["num_heads"] == 4 and spec.layers[0]["mixer"]["num_kv_heads"] == 2
    assert spec.layers[0]["post_mixer_norm"]["eps"] == 0.00001
    assert spec.position_encodings["rope"]["theta"] == 1000000.0
    assert spec.lm_head["tied"] is True


def test_registry_resolves_and_refuses():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert resolve_architecture(raw()).name == "Qwen3ForCausalLM"
    for model_type, names in (("qwen3_moe", ["Qwen3MoeForCausalLM"]), ("llama", ["LlamaForCausalLM"]),
                              ("qwen3", ["Qwen3MoeForCausalLM"]), ("llama", ["Qwen3ForCausalLM"])):
        r = raw()
        r.update(model_type=model_type, architectures=names)
        with pytest.raises(ConfigError, match="unsupported model"):
            resolve_architecture(r)
    by_name = raw()
    del by_name["model_type"]
    assert resolve_architecture(by_name).name == "Qwen3ForCausalLM"
    for broken in ({}, {"model_type": "qwen3"}, {"model_type": 3, "architectures": ["Qwen3ForCausalLM"]}, {"model_type": "qwen3", "architectures": []}, []):
        with pytest.raises(ConfigError):
            resolve_architecture(broken)


def test_registry_takes_a_new_architecture():
    base = resolve_architecture(raw())
    toy = Architecture(name="ToyForCausalLM", model_type="toy", parse_config=base.parse_config,
                       model_spec=base.model_spec, weight_plan=base.weight_plan)
    register_architecture(toy, replace=True)
    with pytest.raises(ValueError):
        register_architecture(toy)
    r = copy.deepcopy(raw())
    r.update(model_type="toy", architectures=["ToyForCausalLM"])
    assert resolve_architecture(r).name == "ToyForCausalLM"


def test_run_list_is_validated():
    from llm_infer_rust_b200 import RunEntry
    import dataclasses
    spec = Qwen3Config.parse(raw()).model_spec()
    for bad in ((RunEntry(0), RunEntry(2)), (RunEntry(0, reads=0),), (RunEntry(0), RunEntry(1, reads=1)),
                (RunEntry(0), RunEntry(1, reads=0), RunEntry(1, reads=1))):
        with pytest.raises(ConfigError):
            dataclasses.replace(spec, run_list=bad).validate()
    dataclasses.replace(spec, run_list=(RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, reads=1))).validate()


def test_generation_config_names_the_stop_ids_first(tmp_path):
    # src/server/components/generation.rs:7-44: generation_config.json's eos_token_id, else config.json's
    import json
    from llm_infer_rust_b200.weights.loader import read_config_json
    r = raw()
    r["eos_token_id"] = 3
    (tmp_path / "config.json").write_text(json.dumps(r))
    assert Qwen3Config.parse(read_config_json(str(tmp_path))).eos_token_ids == (3,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": 0.6}))
    assert Qwen3Config.parse(read_config_json(str(tmp_path))).eos_token_ids == (3,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [5, 4]}))
    assert Qwen3Config.parse(read_config_json(str(tmp_path))).eos_token_ids == (5, 4)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": None}))
    assert Qwen3Config.parse(read_config_json(str(tmp_path))).eos_token_ids == ()
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": r["vocab_size"]}))
    with pytest.raises(ConfigError, match="eos_token_id"):
        Qwen3Config.parse(read_config_json(str(tmp_path)))
    for broken in ("[1, 2]", "{not json"):
        (tmp_path / "generation_config.json").write_text(broken)
        with pytest.raises(ValueError, match="generation_config.json"):
            read_config_json(str(tmp_path))
