"""Fill a model's parameters from a model folder, by tensor name.

dtype rule.  In a bfloat16 engine a floating tensor is kept in bfloat16, except
a tensor that the checkpoint stores in 32-bit (or wider): that one stays
float32, and the part that owns it computes with it as it is.  In a float32
engine every floating tensor becomes float32.  Integer tables become int32.

All faults of a checkpoint are reported at once: one ``WeightError`` lists the
missing tensors, the unexpected ones and those whose shape is wrong (the
reference reports the first missing name or shape only and ignores extras:
src/models/qwen3/model.rs:600-646).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import torch

from .plan import WeightBinding
from .safetensors_io import Checkpoint


class WeightError(RuntimeError):
    def __init__(self, model_dir: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[str]):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"checkpoint in {model_dir} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        super().__init__("\n".join(lines))


def read_config_json(model_dir: str) -> dict:
    """config.json of a model folder.  If the folder also has a generation_config.json with an ``eos_token_id``,
    that one replaces config.json's (the reference's order: src/server/components/generation.rs:7-44)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{model_dir}: no config.json")
    with open(path) as fh:
        config = json.load(fh)
    generation_path = os.path.join(model_dir, "generation_config.json")
    if isinstance(config, dict) and os.path.isfile(generation_path):
        with open(generation_path) as fh:
            try:
                generation = json.load(fh)
            except ValueError as err:
                raise ValueError(f"{generation_path}: not JSON: {err}") from None
        if not isinstance(generation, dict):
            raise ValueError(f"{generation_path}: generation config must be an object")
        if "eos_token_id" in generation:
            config["eos_token_id"] = generation["eos_token_id"]
    return config


def kept_dtype(stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    """The dtype a checkpoint tensor has in memory (see the module's dtype rule)."""
    if not stored.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return engine_dtype


def check_checkpoint(ckpt: Checkpoint, plan: Sequence[WeightBinding], model_dir: str) -> None:
    expected: Dict[str, tuple] = {}
    required = set()
    for binding in plan:
        present = [s.name in ckpt for s in binding.sources]
        for s in binding.sources:
            expected[s.name] = s.shape
        # An optional binding may be wholly absent; a partly present one is missing its rest.
        if not binding.optional or any(present):
            required.update(s.name for s in binding.sources)
    names = set(ckpt.names())
    missing = sorted(required - names)
    unexpected = sorted(names - set(expected))
    wrong = []
    for name in sorted(names & set(expected)):
        _, shape = ckpt.info(name)
        if tuple(shape) != tuple(expected[name]):
            wrong.append(f"{name}: stored {list(shape)}, the model needs {list(expected[name])}")
    if missing or unexpected or wrong:
        raise WeightError(model_dir, missing, unexpected, wrong)


def load_weights(model, plan: Sequence[WeightBinding], model_dir: str,
                 engine_dtype: torch.dtype, device: torch.device) -> List[str]:
    """Check the checkpoint against ``plan`` and bind every parameter of ``model``.

    ``model`` needs ``bind_parameter(path, tensor)`` and ``parameter(path)``.
    Returns the checkpoint tensor names that were loaded.
    """
    ckpt = Checkpoint(model_dir)
    loaded: List[str] = []
    try:
        check_checkpoint(ckpt, plan, model_dir)
        deferred = []
        for binding in plan:
            if binding.optional and not all(s.name in ckpt for s in binding.sources):
                if binding.alias_of is None:
                    continue
                deferred.append(binding)
                continue
            parts = []
            for s in binding.sources:
                t = ckpt.read(s.name)
                parts.append(t)
                loaded.append(s.name)
            # Packed tensors take the widest of their parts' kept dtypes.
            kept = [kept_dtype(t.dtype, engine_dtype) for t in parts]
            dtype = torch.float32 if torch.float32 in kept else kept[0]
            on_device = [t.to(device=device, dtype=dtype, non_blocking=False) for t in parts]
            value = on_device[0] if len(on_device) == 1 else torch.cat(on_device, dim=0)
            model.bind_parameter(binding.param, value.contiguous())
        for binding in deferred:
            model.bind_parameter(binding.param, model.parameter(binding.alias_of))
    finally:
        ckpt.close()
    return loaded
