"""What every part is: a typed bundle of sizes, constants and parameters.

A part is built from a ``PartSpec`` (its sizes and constants) and a ``BuildEnv``
(dtype, device, the model's shared position encodings).  It declares its
parameters by local name and shape; the model gives them dotted paths and the
weight loader binds tensors to them.  No part knows which model it is in.

Categories and the interface each must have:

``norm``              ``forward(x, out=None, rows=None)``,
                      ``forward_add(x, residual, out=None, rows=None, write_residual=True)``
``position_encoding`` attributes that the mixers of the model understand
                      (``half_split_rope``: ``cos``, ``sin``, ``rot_dim``)
``mixer``             ``forward(x, ctx, cache) -> y``; ``cache_spec()`` (paged keys and
                      values it needs, or None); ``state_spec()`` (fixed-size
                      per-request state it needs, or None)
``feed_forward``      ``forward(x) -> y``

Optional, for fusion across parts: a norm may offer ``pending_add(x, residual, ...)``, which
returns the add + norm unrun (``ops.PendingNorm``); a mixer, feed-forward or head that offers
``takes_pending(tokens) -> bool`` and answers True is then given that object as ``x`` and runs it
as the prologue of its first product.  Parts without these methods get plain tensors.
``block``             built from a ``LayerSpec``; ``forward(h, residual, ctx, cache) -> (h, residual)``
``embedding``         ``forward(token_ids) -> h``
``head``              ``forward(x) -> float32 logits``
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..config.spec import PartSpec


@dataclass(frozen=True)
class ParamDecl:
    shape: Tuple[int, ...]
    role: str = "matrix"      # "matrix" | "vector" | "table" (integers)


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of one execution of a mixer, kept in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: all keys are kept; W: only the last W positions are read


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, kept in a slot."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class BuildEnv:
    dtype: torch.dtype                # the engine's activation dtype
    device: torch.device
    position_encodings: Dict[str, "Part"]


class Part:
    category = ""

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec = spec
        self.env = env
        self.params: Dict[str, torch.Tensor] = {}

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {}

    def bind(self, name: str, tensor: torch.Tensor) -> None:
        decl = self.param_decls().get(name)
        if decl is None:
            raise KeyError(f"{type(self).__name__} has no parameter {name!r}")
        if tuple(tensor.shape) != tuple(decl.shape):
            raise ValueError(f"{type(self).__name__}.{name}: shape {tuple(tensor.shape)} "
                             f"does not fit {tuple(decl.shape)}")
        self.params[name] = tensor

    def missing_params(self):
        return [n for n in self.param_decls() if n not in self.params]
