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
    # (tensors that the model does not know refuse nothing by themselves, but the one error lists them)
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


def test_unexpected_tensors_alone_are_ignored(tiny, tmp_path, caplog):
    """A checkpoint with buffers beyond the model's tensors loads (the reference drops the leftover map:
    src/models/qwen3/model.rs:223-265); their number is in the debug log."""
    import logging
    v = tiny["A"]
    d = write_random_model(str(tmp_path), v["raw"], v["seed"])
    w = random_tensors(v["raw"], v["seed"])
    w["model.rotary_emb.inv_freq"] = torch.zeros(8)
    w["extra.bias"] = torch.zeros(3)
    _rewrite(d, w)
    with caplog.at_level(logging.DEBUG, logger="llm_infer_rust_b200"):
        model, loaded = _load(d)
    assert not model.unbound_parameters() and "extra.bias" not in loaded
    assert any("2 tensors that the model does not know are ignored" in r.getMessage() for r in caplog.records)


def test_dtype_rule():
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype(torch.float16, bf) == bf and kept_dtype(bf, bf) == bf
    assert kept_dtype(f32, bf) == bf                          # converted to the engine's dtype ...
    assert kept_dtype(f32, bf, keep_float32=True) == f32      # ... unless the loader says that 32-bit tensors stay
    assert kept_dtype(bf, f32) == f32 and kept_dtype(f32, f32) == f32
    assert kept_dtype(torch.int64, bf) == torch.int32 and kept_dtype(torch.int32, f32) == torch.int32


def _mixed_folder(tiny, tmp_path, declared):
    v = tiny["A"]
    w = {n: t.to(torch.bfloat16) for n, t in random_tensors(v["raw"], v["seed"]).items()}
    w["model.norm.weight"] = w["model.norm.weight"].float()
    w["model.layers.0.self_attn.q_norm.weight"] = w["model.layers.0.self_attn.q_norm.weight"].float()
    with open(tmp_path / "config.json", "w") as fh:
        json.dump(dict(v["raw"], torch_dtype=declared), fh)
    _rewrite(str(tmp_path), w)
    return str(tmp_path)


def test_a_tensor_stored_in_32_bit_in_a_16_bit_checkpoint_stays_so(tiny, tmp_path):
    d = _mixed_folder(tiny, tmp_path, "bfloat16")
    model, _ = _load(d, torch.bfloat16)
    assert model.parameter("final_norm.weight").dtype == torch.float32
    assert model.parameter("layers.0.mixer.q_norm").dtype == torch.float32
    assert model.parameter("layers.0.mixer.k_norm").dtype == torch.bfloat16
    assert model.parameter("layers.1.mixer.qkv_proj").dtype == torch.bfloat16


def test_a_float32_checkpoint_becomes_bfloat16_under_a_bfloat16_engine(tiny, tmp_path, caplog):
    """The reference converts every tensor to the engine's dtype when it binds it (src/models/qwen3/model.rs:616)."""
    import logging
    v = tiny["B"]
    d = write_random_model(str(tmp_path), v["raw"], v["seed"])          # float32 folder, declared float32
    with caplog.at_level(logging.INFO, logger="llm_infer_rust_b200"):
        model, loaded = _load(d, torch.bfloat16)
    shapes = model.parameter_shapes()
    assert all(model.parameter(path).dtype == torch.bfloat16 for path in shapes)
    assert any(f"{len(loaded)} tensors stored in 32-bit were converted to bfloat16" in r.getMessage() for r in caplog.records)
    # the override keeps them, for whoever wants the 32-bit products
    arch = resolve_architecture(v["raw"])
    config = arch.parse_config(v["raw"])
    wide = DecoderModel(arch.model_spec(config), torch.bfloat16, torch.device("cpu"))
    load_weights(wide, arch.weight_plan(config), d, torch.bfloat16, torch.device("cpu"), keep_float32=True)
    assert all(wide.parameter(path).dtype == torch.float32 for path in shapes)


def test_random_values_are_a_function_of_seed_name_and_index():
    """The generator of the random-weights mode, restated in NumPy from its description: two SplitMix64 words per
    element, the sum of their eight 16-bit fields, centred and scaled.  Equal bit for bit, on any cut."""
    import zlib
    import numpy as np
    from llm_infer_rust_b200.weights.random_init import counter_normal

    def mix(x):
        with np.errstate(over="ignore"):
            x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))

    def restated(seed, name, n):
        with np.errstate(over="ignore"):
            key = mix(mix(np.uint64(seed)) ^ (np.uint64(zlib.crc32(name.encode())) * np.uint64(0x9E3779B97F4A7C15)))
            i = np.arange(n, dtype=np.uint64)
            total = np.zeros(n, dtype=np.int64)
            for word in (0, 1):
                h = mix(key + i * np.uint64(2) + np.uint64(word))
                for field in range(4):
                    total += ((h >> np.uint64(16 * field)) & np.uint64(0xFFFF)).astype(np.int64)
        scale = np.float32(1.0 / np.sqrt(8 * (65536.0 ** 2 - 1.0) / 12.0))
        return (total.astype(np.float32) - np.float32(8 * 32767.5)) * scale

    for seed, name, shape in ((0, "model.embed_tokens.weight", (7, 13)), (5, "model.layers.3.mlp.up_proj.weight", (1000,))):
        got = counter_normal(seed, name, shape)
        want = restated(seed, name, got.numel())
        assert np.array_equal(got.view(-1).numpy(), want)
    big = counter_normal(1, "x", (200000,))
    assert abs(big.mean().item()) < 0.01 and abs(big.std().item() - 1.0) < 0.01
    assert not torch.equal(counter_normal(1, "x", (64,)), counter_normal(1, "y", (64,)))


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
