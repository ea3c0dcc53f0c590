"""Typed configuration of dense Qwen3, read from its own config.json keys.

Accept / reject rules follow the reference (src/models/qwen3/config.rs:63-185):
derived defaults for ``num_key_value_heads`` and ``head_dim``, fixed defaults
for ``max_position_embeddings`` (8192), ``rope_theta`` (10000), ``rms_norm_eps``
(1e-6) and ``tie_word_embeddings`` (false); unsupported computation features
are refused before anything is loaded.

One deliberate widening: the reference refuses ``use_sliding_window`` and any
``layer_types`` entry other than ``"full_attention"`` (config.rs:105-126).  The
attention part and the cache manager here take a window as a parameter, so
``use_sliding_window: true`` with ``sliding_window: W`` is accepted; the layers
that use it are given by ``layer_types`` (``"sliding_attention"``) or, without
it, are those with index >= ``max_window_layers``.  A query at position p then
sees the keys j with p - W < j <= p.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

_I64_MAX = 2 ** 63 - 1


def _positive_int(raw: dict, key: str, default: Optional[int] = None) -> int:
    if key not in raw:
        if default is None:
            raise ConfigError(f"missing {key}")
        return default
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"invalid {key}: {value!r} (an integer is required)")
    if value <= 0 or value > _I64_MAX:
        raise ConfigError(f"{key} must be positive and fit in i64")
    return value


def _positive_float(raw: dict, key: str, default: float) -> float:
    if key not in raw:
        return default
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"invalid {key}: {value!r} (a number is required)")
    value = float(value)
    if not math.isfinite(value) or value <= 0.0:
        raise ConfigError(f"{key} must be positive and finite")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    layer_windows: Tuple[Optional[int], ...]   # per layer: window length or None
    checkpoint_dtype: str                      # "float32" | "float16" | "bfloat16"
    eos_token_ids: Tuple[int, ...]

    model_type = "qwen3"
    architecture = "Qwen3ForCausalLM"

    @staticmethod
    def parse(raw: Any) -> "Qwen3Config":
        if not isinstance(raw, dict):
            raise ConfigError("config must be an object")
        for key in ("rope_scaling", "rope_parameters", "quantization_config", "compression_config"):
            if raw.get(key) is not None:
                raise ConfigError(f"unsupported Qwen3 computation feature: {key}")
        for key in ("attention_bias", "mlp_bias"):
            if key in raw and raw[key] is not False:
                raise ConfigError(f"unsupported or invalid Qwen3 {key}: {raw[key]!r}")
        if "hidden_act" in raw and raw["hidden_act"] != "silu":
            raise ConfigError(f"unsupported Qwen3 hidden_act: {raw['hidden_act']!r}")
        if "qk_norm" in raw and raw["qk_norm"] is not True:
            raise ConfigError("Qwen3 requires qk_norm=true")

        hidden = _positive_int(raw, "hidden_size")
        layers = _positive_int(raw, "num_hidden_layers")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = _positive_int(raw, "num_key_value_heads", heads)
        if "head_dim" in raw:
            head_dim = _positive_int(raw, "head_dim")
        else:
            if hidden % heads != 0:
                raise ConfigError("hidden_size must be divisible by num_attention_heads "
                                  "when head_dim is omitted")
            head_dim = hidden // heads
        inter = _positive_int(raw, "intermediate_size")
        vocab = _positive_int(raw, "vocab_size")
        max_pos = _positive_int(raw, "max_position_embeddings", 8192)
        theta = _positive_float(raw, "rope_theta", 10000.0)
        eps = _positive_float(raw, "rms_norm_eps", 1e-6)
        tie = raw.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise ConfigError(f"invalid tie_word_embeddings: {tie!r} (true or false is required)")
        if heads % kv_heads != 0:
            raise ConfigError("num_attention_heads must be divisible by num_key_value_heads")
        if head_dim % 2 != 0:
            raise ConfigError("Qwen3 RoPE requires an even head_dim")
        for width in ((heads + 2 * kv_heads) * head_dim, 2 * inter):
            if width > _I64_MAX:
                raise ConfigError("Qwen3 projection width exceeds i64")

        windows = Qwen3Config._windows(raw, layers)
        dtype = raw.get("torch_dtype", raw.get("dtype", "float32"))
        if dtype not in ("float32", "float16", "bfloat16"):
            raise ConfigError(f"unsupported checkpoint dtype: {dtype!r}")
        return Qwen3Config(hidden, layers, heads, kv_heads, head_dim, inter, vocab, max_pos,
                           theta, eps, tie, windows, dtype,
                           Qwen3Config._eos(raw.get("eos_token_id"), vocab))

    @staticmethod
    def _windows(raw: dict, layers: int) -> Tuple[Optional[int], ...]:
        use = raw.get("use_sliding_window", False)
        if not isinstance(use, bool):
            raise ConfigError(f"unsupported or invalid Qwen3 use_sliding_window: {use!r}")
        types = raw.get("layer_types")
        if types is not None:
            if not isinstance(types, list) or len(types) != layers or any(
                    t not in ("full_attention", "sliding_attention") for t in types):
                raise ConfigError("invalid layer_types: one of full_attention / sliding_attention "
                                  "is required for every layer")
        if not use:
            # A dormant sliding_window value is metadata; a layer that asks for one is not.
            if types is not None and any(t != "full_attention" for t in types):
                raise ConfigError("layer_types asks for sliding_attention but "
                                  "use_sliding_window is false")
            return tuple([None] * layers)
        window = _positive_int(raw, "sliding_window")
        if types is not None:
            return tuple(window if t == "sliding_attention" else None for t in types)
        first = raw.get("max_window_layers", 0)
        if isinstance(first, bool) or not isinstance(first, int) or first < 0:
            raise ConfigError(f"invalid max_window_layers: {first!r}")
        return tuple(window if i >= first else None for i in range(layers))

    @staticmethod
    def _eos(value: Any, vocab: int) -> Tuple[int, ...]:
        # src/server/components/generation.rs:7-69: an int, a list of ints, or null / [] for none.
        if value is None:
            return ()
        ids = value if isinstance(value, list) else [value]
        for i in ids:
            if isinstance(i, bool) or not isinstance(i, int) or not 0 <= i < vocab:
                raise ConfigError(f"invalid eos_token_id: {i!r}")
        return tuple(ids)

    # ------------------------------------------------------------------ parts
    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm", {"width": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("half_split_rope", {"rotary_dim": self.head_dim, "theta": self.rope_theta,
                                            "max_positions": self.max_position_embeddings})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                  "intermediate_size": self.intermediate_size})
        layers = []
        for window in self.layer_windows:
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                "qk_norm_eps": self.rms_norm_eps, "window": window,
                "softmax_scale": 1.0 / math.sqrt(self.head_dim), "position_encoding": "rope"})
            layers.append(LayerSpec.pre_norm(PartSpec("pre_norm_deferred_add"), mixer, ffn, norm))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size,
            hidden_size=self.hidden_size, max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size,
                                                   "hidden_size": self.hidden_size}),
            layers=tuple(layers),
            run_list=tuple(RunEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=norm,
            lm_head=PartSpec("linear_head", {"vocab_size": self.vocab_size,
                                             "hidden_size": self.hidden_size,
                                             "tied": self.tie_word_embeddings}),
            position_encodings={"rope": rope})
        spec.validate()
        return spec
