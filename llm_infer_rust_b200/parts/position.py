"""Position encodings."""
from __future__ import annotations

import math

import torch

from .base import Part
from .registry import register_part


class HalfSplitRope(Part):
    """Rotary tables for the half-split ("rotate_half") layout.

    angle[p, i] = p * theta^(-2i / rot_dim), i in [0, rot_dim / 2); the pair
    (i, i + rot_dim / 2) of a head is rotated by it (reference:
    src/layers/ops.rs:70-127, which builds the table in float32 on the GPU).
    The angles are computed in float64 and the cosines and sines stored as
    float32 [max_positions, rot_dim / 2]; the rotation itself runs in float.
    """
    category = "position_encoding"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.rot_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        if self.rot_dim % 2:
            raise ValueError("rotary_dim must be even")
        i = torch.arange(0, self.rot_dim, 2, dtype=torch.float64)
        inv_freq = torch.exp(i * (-(math.log(self.theta) / self.rot_dim)))
        angle = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.cos = torch.cos(angle).to(torch.float32).to(env.device).contiguous()
        self.sin = torch.sin(angle).to(torch.float32).to(env.device).contiguous()


register_part("position_encoding", "half_split_rope", HalfSplitRope)
