"""One registry from an architecture's name to everything that builds it.

The reference keeps a static table keyed by (model_type, architectures)
(src/models/registry.rs:19-38) and refuses an unknown model before anything is
loaded (src/server/components/builder.rs:111-120).  Here the table can grow at
run time: ``register_architecture`` is all that a new architecture needs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Sequence

from .spec import ConfigError, ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str                                     # e.g. "Qwen3ForCausalLM"
    model_type: str                               # config.json "model_type"
    parse_config: Callable[[dict], Any]           # raw config.json -> typed configuration
    model_spec: Callable[[Any], ModelSpec]        # typed configuration -> parts and run list
    weight_plan: Callable[[Any], List[Any]]       # typed configuration -> WeightBinding list
    # typed configuration -> the dtype its checkpoint declares ("float32", "bfloat16", "float16"): the engine's "auto"
    checkpoint_dtype: Callable[[Any], str] = lambda config: "bfloat16"
    # typed configuration -> token ids that end a generation
    stop_ids: Callable[[Any], Sequence[int]] = lambda config: ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name} is already registered")
    _ARCHITECTURES[arch.name] = arch


def registered_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw_config: dict) -> Architecture:
    if not isinstance(raw_config, dict):
        raise ConfigError("config must be an object")
    names = raw_config.get("architectures")
    model_type = raw_config.get("model_type")
    if not isinstance(names, list) or not names or not (model_type is None or isinstance(model_type, str)):
        raise ConfigError("config.json needs a non-empty architectures list (and model_type, a string)")
    # The architecture's name selects; a model_type that is given must agree with it (the reference
    # wants both keys; a folder written without model_type is still named unambiguously).
    for name in names:
        arch = _ARCHITECTURES.get(name)
        if arch is not None and (model_type is None or arch.model_type == model_type):
            return arch
    raise ConfigError(f"unsupported model: model_type={model_type!r}, architectures={names!r}; "
                      f"registered: {registered_architectures()}")
