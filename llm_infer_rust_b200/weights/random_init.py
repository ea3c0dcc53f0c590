"""Random-weights mode: write a model folder from a configuration and a seed, or fill a model on the device.

The reference has no such mode (its parameters start as zeros and its tests
fill them by hand: src/models/qwen3/model.rs:595-597, :749-780).  Here a folder
with ``config.json`` and ``model.safetensors`` is written, so that everything
downstream (registry, loader, engine, trace replay) runs exactly as it does for
a real checkpoint; for sizes whose folder would take long to write the same
values are drawn on the device without a file (``bind_random_weights``).

Matrices are N(0, std); norm weights are 1 + N(0, norm_std) (norm_std 0 gives
ones).  Every value is a function of (seed, tensor name, element index) alone:
a counter-based generator in integer arithmetic, so a tensor does not depend on
which other tensors exist, on the device that draws it, or on how the draw is
cut into pieces, and a few lines of NumPy reproduce any element (the tests do).

The generator.  key = 64-bit mix of (seed, CRC-32 of the name).  For element i
two 64-bit words h1 = mix(key + i * 2), h2 = mix(key + i * 2 + 1) (``mix``: the
finalizer of SplitMix64) give eight 16-bit fields; their sum S is an
Irwin-Hall variate, and z = (S - 8 * 32767.5) / sqrt(8 * (65536^2 - 1) / 12) is
the standard normal value used (bounded at 4.9 sigma).  The integer part is
exact everywhere; the float32 part is one subtraction and one multiplication.
"""
from __future__ import annotations

import json
import math
import os
import zlib
from typing import Dict, Optional

import torch

from ..config.registry import resolve_architecture
from .safetensors_io import write_safetensors

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}
_MASK = (1 << 64) - 1
_NORMAL_SCALE = 1.0 / math.sqrt(8 * (65536.0 ** 2 - 1.0) / 12.0)
_CHUNK = 1 << 24                 # elements drawn at a time (bounds the temporaries of a large tensor)


def _mix_int(x: int) -> int:
    """SplitMix64's finalizer on a Python integer."""
    x &= _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def _signed(x: int) -> int:
    return x - (1 << 64) if x >= (1 << 63) else x


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of one tensor's stream."""
    return _mix_int(_mix_int(int(seed)) ^ (zlib.crc32(name.encode()) * 0x9E3779B97F4A7C15))


def _srl(x: torch.Tensor, bits: int) -> torch.Tensor:
    """Logical right shift of int64 (torch's is arithmetic)."""
    return (x >> bits) & ((1 << (64 - bits)) - 1)


def _mix(x: torch.Tensor) -> torch.Tensor:
    """SplitMix64's finalizer on int64 tensors (products wrap modulo 2^64)."""
    x = (x ^ _srl(x, 30)) * _signed(0xBF58476D1CE4E5B9)
    x = (x ^ _srl(x, 27)) * _signed(0x94D049BB133111EB)
    return x ^ _srl(x, 31)


def counter_normal(seed: int, name: str, shape, device="cpu") -> torch.Tensor:
    """float32 standard-normal values of the tensor ``name`` (see the module's header), on ``device``."""
    n = 1
    for s in shape:
        n *= int(s)
    key = _signed(tensor_key(seed, name))
    out = torch.empty(n, dtype=torch.float32, device=device)
    for at in range(0, n, _CHUNK):
        i = torch.arange(at, min(n, at + _CHUNK), dtype=torch.int64, device=device)
        total = torch.zeros_like(i)
        for word in (0, 1):
            h = _mix(key + i * 2 + word)
            for field in range(4):
                total += _srl(h, 16 * field) & 0xFFFF
        out[at:at + i.numel()] = (total.to(torch.float32) - 8 * 32767.5) * _NORMAL_SCALE
    return out.view(*[int(s) for s in shape])


def _draw(src, seed: int, std: float, norm_std: float, device) -> torch.Tensor:
    """One checkpoint tensor in float32 (integer tables in int32)."""
    if src.integer:
        key = _signed(tensor_key(seed, src.name))
        n = 1
        for s in src.shape:
            n *= int(s)
        i = torch.arange(n, dtype=torch.int64, device=device)
        return (_srl(_mix(key + i), 49)).to(torch.int32).view(*src.shape)          # 15 bits
    z = counter_normal(seed, src.name, src.shape, device)
    if src.init == "norm":
        return 1.0 + norm_std * z if norm_std else torch.ones_like(z)
    return std * z


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
            value = _draw(src, seed, std, norm_std, "cpu")
            tensors[src.name] = value if src.integer else value.to(store)
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
    """Fill ``model`` with the weights that ``random_tensors`` gives for the same seed, drawn on ``device``
    (float32 values, rounded once to ``engine_dtype``); nothing is written or read.
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
            value = _draw(src, seed, std, norm_std, device)
            parts.append(value if src.integer else value.to(engine_dtype))
            names.append(src.name)
        model.bind_parameter(binding.param, parts[0] if len(parts) == 1 else torch.cat(parts, dim=0))
    for binding in deferred:
        model.bind_parameter(binding.param, model.parameter(binding.alias_of))
    return names
