"""Safetensors reading and writing, the loader's dtype rule and its one error."""
import json
import os

import pytest
import torch

from llm_infer_rust_b200 import random_tensors, resolve_architecture, write_random_model
from llm_infer_rust_b200.parts import DecoderModel
from llm_infer_rust_b200.weights import (Checkpoint, SafetensorsError, WeightError, kept_dtype, load_weights,
                                         write_safetensors)


def _load(model_dir, dtype=torch.float32):
    with open(os.path.join(model_dir, "config.json")) as fh:
        raw = json.load(fh)
    arch = resolve_architecture(raw)
    config = arch.parse_config(raw)
    model = DecoderModel(arch.model_spec(config), dtype, torch.device("cpu"))
    loaded = load_weights(model, arch.weight_plan(config), model_dir, dtype, torch.device("cpu"))
    return model, loaded


def _rewrite(model_dir, tensors):
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors.items())


def test_round_trip_of_the_container(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).view(2, 3), "empty": torch.zeros(0, 4)}
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    ck = Checkpoint(str(tmp_path))
    assert sorted(ck.names()) == sorted(tensors)
    for name, t in tensors.items():
        got = ck.read(name)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t)
    ck.close()


def test_random_model_folder_loads_and_counts(tiny, tmp_path):
    v = tiny["B"]
    d = write_random_model(str(tmp_path), v["raw"], v["seed"], norm_std=v["norm_std"])
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    model, loaded = _load(d)
    layers = v["raw"]["num_hidden_layers"]
    assert len(loaded) == 11 * layers + 3            # untied: embedding, final norm, head
    assert not model.unbound_parameters()
    w = random_tensors(v["raw"], v["seed"], norm_std=v["norm_std"])
    qkv = model.parameter("layers.1.mixer.qkv_proj")
    want = torch.cat([w[f"model.layers.1.self_attn.{n}_proj.weight"] for n in "qkv"])
    assert torch.equal(qkv, want)
    gu = model.parameter("layers.2.feed_forward.gate_up_proj")
    assert torch.equal(gu, torch.cat([w["model.layers.2.mlp.gate_proj.weight"],
                                      w["model.layers.2.mlp.up_proj.weight"]]))


def test_same_seed_same_weights_other_seed_other_weights(tiny):
    raw = tiny["A"]["raw"]
    a, b, c = random_tensors(raw, 3), random_tensors(raw, 3), random_tensors(raw, 4)
    assert all(torch.equal(a[n], b[n]) for n in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert torch.equal(a["model.norm.weight"], torch.ones_like(a["model.norm.weight"]))
    assert abs(a["model.embed_tokens.weight"].std().item() - 0.02) < 0.002


def test_tied_head_aliases_the_embedding_and_a_stored_head_wins(tiny, tmp_path):
    v = tiny["A"]
    d = write_random_model(str(tmp_path), v["raw"], v["seed"])
    model, loaded = _load(d)
    assert "lm_head.weight" not in loaded
    assert model.parameter("lm_head.weight").data_ptr() == model.parameter("embedding.weight").data_ptr()
    w = random_tensors(v["raw"], v["seed"])
    w["lm_head.weight"] = torch.randn(v["raw"]["vocab_size"], v["raw"]["hidden_size"])
    _rewrite(d, w)
    model, loaded = _load(d)
    assert "lm_head.weight" in loaded
    assert torch.equal(model.parameter("lm_head.weight"), w["lm_head.weight"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tiny, tmp_path):
    v = tiny["B"]
    d = write_random_model(str(tmp_path), v["raw"], v["seed"])
    w = random_tensors(v["raw"], v["seed"])
    del w["model.layers.0.self_attn.k_proj.weight"]
    del w["lm_head.weight"]                                   # untied: it is required
    w["model.layers.1.mlp.down_proj.weight"] = torch.zeros(5, 5)
    w["model.layers.2.self_attn.q_norm.weight"] = torch.zeros(v["raw"]["head_dim"] + 1)
    w["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    w["extra.bias"] = torch.zeros(3)
    _rewrite(d, w)
    with pytest.raises(WeightError) as info:
        _load(d)
    err = info.value
    assert err.missing == ["lm_head.weight", "model.layers.0.self_attn.k_proj.weight"]
    assert err.unexpected == ["extra.bias", "model.layers.7.mlp.up_proj.weight"]
    assert len(err.wrong_shape) == 2 and "down_proj" in err.wrong_shape[0] and "[5, 5]" in err.wrong_shape[0]
    text = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (2)", "extra.bias",
                   "k_proj", "q_norm"):
        assert needle in text


def test_dtype_rule():
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype(torch.float16, bf) == bf and kept_dtype(bf, bf) == bf
    assert kept_dtype(f32, bf) == f32                         # stored in 32-bit: stays so
    assert kept_dtype(bf, f32) == f32 and kept_dtype(f32, f32) == f32
    assert kept_dtype(torch.int64, bf) == torch.int32 and kept_dtype(torch.int32, f32) == torch.int32


def test_a_tensor_stored_in_32_bit_stays_so_in_a_bfloat16_model(tiny, tmp_path):
    v = tiny["A"]
    w = {n: t.to(torch.bfloat16) for n, t in random_tensors(v["raw"], v["seed"]).items()}
    w["model.norm.weight"] = w["model.norm.weight"].float()
    w["model.layers.0.self_attn.q_norm.weight"] = w["model.layers.0.self_attn.q_norm.weight"].float()
    with open(tmp_path / "config.json", "w") as fh:
        json.dump(v["raw"], fh)
    _rewrite(str(tmp_path), w)
    model, _ = _load(str(tmp_path), torch.bfloat16)
    assert model.parameter("final_norm.weight").dtype == torch.float32
    assert model.parameter("layers.0.mixer.q_norm").dtype == torch.float32
    assert model.parameter("layers.0.mixer.k_norm").dtype == torch.bfloat16
    assert model.parameter("layers.1.mixer.qkv_proj").dtype == torch.bfloat16


def test_shards_duplicates_and_unsafe_paths(tiny, tmp_path):
    v = tiny["A"]
    w = random_tensors(v["raw"], v["seed"])
    names = sorted(w)
    first, second = names[: len(names) // 2], names[len(names) // 2:]
    write_safetensors(str(tmp_path / "s1.safetensors"), [(n, w[n]) for n in first])
    write_safetensors(str(tmp_path / "s2.safetensors"), [(n, w[n]) for n in second])
    index = {"weight_map": {**{n: "s1.safetensors" for n in first}, **{n: "s2.safetensors" for n in second}}}
    with open(tmp_path / "model.safetensors.index.json", "w") as fh:
        json.dump(index, fh)
    with open(tmp_path / "config.json", "w") as fh:
        json.dump(v["raw"], fh)
    model, loaded = _load(str(tmp_path))
    assert sorted(loaded) == names
    # the same tensor in two shards
    write_safetensors(str(tmp_path / "s2.safetensors"), [(n, w[n]) for n in second + first[:1]])
    with pytest.raises(SafetensorsError, match="both"):
        _load(str(tmp_path))
    for bad in ("../x.safetensors", "/abs/x.safetensors"):
        with open(tmp_path / "model.safetensors.index.json", "w") as fh:
            json.dump({"weight_map": {"a": bad}}, fh)
        with pytest.raises(SafetensorsError, match="leaves the model folder"):
            _load(str(tmp_path))
    with open(tmp_path / "model.safetensors.index.json", "w") as fh:
        fh.write("{not json")
    with pytest.raises(SafetensorsError, match="invalid index"):
        _load(str(tmp_path))
    os.remove(tmp_path / "model.safetensors.index.json")
    with pytest.raises(SafetensorsError, match="neither"):
        _load(str(tmp_path))


def test_a_truncated_file_is_refused(tmp_path):
    write_safetensors(str(tmp_path / "model.safetensors"), [("a", torch.randn(64, 64))])
    path = tmp_path / "model.safetensors"
    data = path.read_bytes()
    path.write_bytes(data[: len(data) // 2])
    with pytest.raises(SafetensorsError, match="inconsistent offsets"):
        Checkpoint(str(tmp_path))


def test_malformed_headers_are_refused_with_the_container_error(tmp_path):
    import struct
    path = tmp_path / "model.safetensors"

    def stored(header, data=b"\0" * 16):
        text = header if isinstance(header, bytes) else json.dumps(header).encode()
        path.write_bytes(struct.pack("<Q", len(text)) + text + data)

    good = {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}
    stored(good)
    assert Checkpoint(str(tmp_path)).read("a").shape == (2, 2)
    for header, what in (
            (b"{not json", "not JSON"), ([1, 2], "not a JSON object"),
            ({"a": {"dtype": "F32", "shape": [2, 2]}}, "malformed"),
            ({"a": [1, 2, 3]}, "malformed"),
            ({"a": {"dtype": "F32", "shape": [2, "2"], "data_offsets": [0, 16]}}, "malformed"),
            ({"a": {"dtype": "F32", "shape": [-2, -2], "data_offsets": [0, 16]}}, "malformed"),
            ({"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0]}}, "malformed"),
            ({"a": {"dtype": "F8_E4M3", "shape": [16], "data_offsets": [0, 16]}}, "unsupported dtype"),
            ({"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [4, 16]}}, "inconsistent offsets"),
            ({"a": {"dtype": "F32", "shape": [2, 4], "data_offsets": [0, 32]}}, "inconsistent offsets")):
        stored(header)
        with pytest.raises(SafetensorsError, match=what):
            Checkpoint(str(tmp_path))
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds the file"):
        Checkpoint(str(tmp_path))
    path.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        Checkpoint(str(tmp_path))
