"""Fill a model's parameters from a model folder, by tensor name.

dtype rule.  In a float32 engine every floating tensor becomes float32; integer
tables become int32.  In a bfloat16 engine floating tensors become bfloat16,
with one exception: a tensor that a 16-bit checkpoint (``torch_dtype`` bfloat16
or float16 in its config.json) stores in 32-bit stays float32, and the part that
owns it computes with it as it is; such a tensor was widened on purpose.  A
checkpoint that is 32-bit as a whole is converted like any other (the
reference converts every tensor to the engine's dtype when it binds it:
src/models/qwen3/model.rs:616, :642).  ``keep_float32`` overrides the rule:
True keeps every 32-bit tensor, False keeps none.

Faults of a checkpoint are reported at once: one ``WeightError`` lists the
missing tensors and those whose shape is wrong, and with them the tensors of
the file that the model does not know (an unexpected name often explains a
missing one).  Unexpected tensors alone refuse nothing: they are ignored, as in
the reference (src/engine/model_loader.rs:108-122; the leftover map is dropped,
src/models/qwen3/model.rs:223-265), and counted in the log.
"""
from __future__ import annotations

import json
import logging
import os
from typing import Dict, List, Optional, Sequence

import torch

from .plan import WeightBinding
from .safetensors_io import Checkpoint


log = logging.getLogger("llm_infer_rust_b200")


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


def kept_dtype(stored: torch.dtype, engine_dtype: torch.dtype, keep_float32: bool = False) -> torch.dtype:
    """The dtype a checkpoint tensor has in memory; ``keep_float32``: 32-bit tensors stay so under a 16-bit engine
    (see the module's dtype rule for when the loader says so)."""
    if not stored.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if keep_float32 and stored in (torch.float32, torch.float64):
        return torch.float32
    return engine_dtype


def checkpoint_is_16_bit(model_dir: str) -> bool:
    """Whether config.json declares a 16-bit checkpoint (``torch_dtype`` or ``dtype``)."""
    try:
        with open(os.path.join(model_dir, "config.json")) as fh:
            raw = json.load(fh)
    except (OSError, ValueError):
        return False
    declared = raw.get("torch_dtype", raw.get("dtype")) if isinstance(raw, dict) else None
    return declared in ("bfloat16", "float16")


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
    if missing or wrong:
        raise WeightError(model_dir, missing, unexpected, wrong)
    if unexpected:
        log.debug("%s: %d tensors that the model does not know are ignored: %s", model_dir, len(unexpected),
                  ", ".join(unexpected[:8]) + (" ..." if len(unexpected) > 8 else ""))


def load_weights(model, plan: Sequence[WeightBinding], model_dir: str,
                 engine_dtype: torch.dtype, device: torch.device, keep_float32: Optional[bool] = None) -> List[str]:
    """Check the checkpoint against ``plan`` and bind every parameter of ``model``.

    ``model`` needs ``bind_parameter(path, tensor)`` and ``parameter(path)``.
    ``keep_float32``: None applies the module's dtype rule, True / False override it.
    Returns the checkpoint tensor names that were loaded.
    """
    ckpt = Checkpoint(model_dir)
    loaded: List[str] = []
    if keep_float32 is None:
        keep_float32 = checkpoint_is_16_bit(model_dir)
    kept_wide, narrowed = 0, 0
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
            kept = [kept_dtype(t.dtype, engine_dtype, keep_float32) for t in parts]
            dtype = torch.float32 if torch.float32 in kept else kept[0]
            wide = sum(t.dtype in (torch.float32, torch.float64) for t in parts)
            if engine_dtype != torch.float32 and wide:
                kept_wide += wide if dtype == torch.float32 else 0
                narrowed += 0 if dtype == torch.float32 else wide
            on_device = [t.to(device=device, dtype=dtype, non_blocking=False) for t in parts]
            value = on_device[0] if len(on_device) == 1 else torch.cat(on_device, dim=0)
            model.bind_parameter(binding.param, value.contiguous())
        for binding in deferred:
            model.bind_parameter(binding.param, model.parameter(binding.alias_of))
    finally:
        ckpt.close()
    if narrowed:
        log.info("%s: %d tensors stored in 32-bit were converted to %s, the engine's dtype", model_dir, narrowed,
                 str(engine_dtype).replace("torch.", ""))
    if kept_wide:
        log.info("%s: %d tensors stored in 32-bit stay float32 (their owners compute in 32-bit)", model_dir, kept_wide)
    return loaded
