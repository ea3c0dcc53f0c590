"""How checkpoint tensors map to the parameters of the parts: pure data.

An architecture returns a list of ``WeightBinding``.  The loader uses it to
check a checkpoint (missing, unexpected, wrong shape) and to fill the model;
the random-weights writer uses it to know which tensors a model folder holds.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class SourceTensor:
    name: str                     # tensor name in the checkpoint
    shape: Tuple[int, ...]
    init: str = "matrix"          # random-weights rule: "matrix" N(0, std) | "norm" 1 + N(0, norm_std)
    integer: bool = False         # an integer table (kept as int32)


@dataclass(frozen=True)
class WeightBinding:
    param: str                                # parameter path in the model, e.g. "layers.3.mixer.qkv_proj"
    sources: Tuple[SourceTensor, ...]         # concatenated along dim 0, in this order
    optional: bool = False                    # the checkpoint may leave it out ...
    alias_of: Optional[str] = None            # ... and then this parameter shares the storage of that one
