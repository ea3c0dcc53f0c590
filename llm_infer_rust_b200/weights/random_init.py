"""Random-weights mode: write a model folder from a configuration and a seed.

The reference has no such mode (its parameters start as zeros and its tests
fill them by hand: src/models/qwen3/model.rs:595-597, :749-780).  Here a folder
with ``config.json`` and ``model.safetensors`` is written, so that everything
downstream (registry, loader, engine, trace replay) runs exactly as it does for
a real checkpoint.

Matrices are N(0, std); norm weights are 1 + N(0, norm_std) (norm_std 0 gives
ones).  Each tensor has a generator of its own, seeded from (seed, tensor
name), so a tensor's values do not depend on which other tensors exist.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Optional

import torch

from ..config.registry import resolve_architecture
from .safetensors_io import write_safetensors

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _generator(seed: int, name: str) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed((int(seed) * 1_000_003 + zlib.crc32(name.encode())) % (2 ** 63 - 1))
    return g


def random_tensors(raw_config: dict, seed: int, std: float = 0.02, norm_std: float = 0.0,
                   dtype: Optional[str] = None) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors (by checkpoint name) for ``raw_config``.

    With tied embeddings no separate head is written.
    """
    arch = resolve_architecture(raw_config)
    config = arch.parse_config(raw_config)
    store = _TORCH_DTYPES[dtype or raw_config.get("torch_dtype", "float32")]
    tensors: Dict[str, torch.Tensor] = {}
    for binding in arch.weight_plan(config):
        if binding.optional and binding.alias_of is not None:
            continue
        for src in binding.sources:
            g = _generator(seed, src.name)
            if src.integer:
                value = torch.randint(0, 2 ** 15, src.shape, generator=g, dtype=torch.int32)
            elif src.init == "norm":
                value = 1.0 + norm_std * torch.randn(src.shape, generator=g, dtype=torch.float32)
                value = value.to(store)
            else:
                value = (std * torch.randn(src.shape, generator=g, dtype=torch.float32)).to(store)
            tensors[src.name] = value
    return tensors


def write_random_model(model_dir: str, raw_config: dict, seed: int, std: float = 0.02,
                       norm_std: float = 0.0, dtype: Optional[str] = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` into ``model_dir``."""
    os.makedirs(model_dir, exist_ok=True)
    config = dict(raw_config)
    if dtype is not None:
        config["torch_dtype"] = dtype
    config.setdefault("torch_dtype", "float32")
    tensors = random_tensors(config, seed, std, norm_std, config["torch_dtype"])
    with open(os.path.join(model_dir, "config.json"), "w") as fh:
        json.dump(config, fh, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors.items())
    return model_dir


def bind_random_weights(model, plan, seed: int, engine_dtype: torch.dtype, device: torch.device,
                        std: float = 0.02, norm_std: float = 0.0):
    """Fill ``model`` with random weights drawn on ``device``; nothing is written or read.

    Same distributions as ``random_tensors`` (the values differ: the device's generator draws them).
    Returns the checkpoint names that a folder of this model would hold.
    """
    names = []
    deferred = []
    for binding in plan:
        if binding.optional and binding.alias_of is not None:
            deferred.append(binding)
            continue
        parts = []
        for src in binding.sources:
            g = torch.Generator(device=device)
            g.manual_seed((int(seed) * 1_000_003 + zlib.crc32(src.name.encode())) % (2 ** 63 - 1))
            if src.integer:
                value = torch.randint(0, 2 ** 15, src.shape, generator=g, dtype=torch.int32, device=device)
            elif src.init == "norm":
                value = (1.0 + norm_std * torch.randn(src.shape, generator=g, dtype=torch.float32,
                                                      device=device)).to(engine_dtype)
            else:
                value = torch.randn(src.shape, generator=g, dtype=engine_dtype, device=device).mul_(std)
            parts.append(value)
            names.append(src.name)
        model.bind_parameter(binding.param, parts[0] if len(parts) == 1 else torch.cat(parts, dim=0))
    for binding in deferred:
        model.bind_parameter(binding.param, model.parameter(binding.alias_of))
    return names
