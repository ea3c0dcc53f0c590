"""Sampling options and the sampler that turns logits into token ids.

Options and their meaning follow the reference (src/engine/sampling.rs:9-48):
``temperature`` (<= 0: greedy), ``top_k`` (<= 0: off), ``top_p`` (0: greedy,
outside [0, 1]: 1), ``ignore_eos``, ``max_tokens`` (at least 1).  ``seed`` is
this engine's addition: the uniform number of a draw is a counter-based random
number keyed by (seed, index of the output token), so a request samples the same
tokens whatever else shares its batch.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import ops

ROW_DTYPE = np.dtype([("temperature", "<f4"), ("top_k", "<i4"), ("top_p", "<f4"), ("seed_lo", "<u4"),
                      ("seed_hi", "<u4"), ("counter", "<u4"), ("pad0", "<i4"), ("pad1", "<i4")])
assert ROW_DTYPE.itemsize == 32


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    ignore_eos: bool = False
    max_tokens: int = 1024
    seed: Optional[int] = None

    def normalized(self) -> "SamplingParams":
        top_p = self.top_p if (math.isfinite(self.top_p) and 0.0 <= self.top_p <= 1.0) else 1.0
        return SamplingParams(float(self.temperature), int(self.top_k), float(top_p),
                              bool(self.ignore_eos), max(int(self.max_tokens), 1), self.seed)

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0) or self.top_p == 0.0


def pack_rows(rows: Sequence[Tuple[SamplingParams, int, int]]) -> np.ndarray:
    """(params, seed, counter) per row -> the 32-byte records that the kernel reads."""
    out = np.zeros(len(rows), dtype=ROW_DTYPE)
    for i, (p, seed, counter) in enumerate(rows):
        seed &= (1 << 64) - 1
        out[i] = (p.temperature, p.top_k, p.top_p, seed & 0xFFFFFFFF, seed >> 32,
                  counter & 0xFFFFFFFF, 0, 0)
    return out


class Sampler:
    def __init__(self, device: torch.device):
        self.device = torch.device(device)

    def sample_device(self, logits: torch.Tensor,
                      rows: Sequence[Tuple[SamplingParams, int, int]]) -> torch.Tensor:
        """int32 token ids [rows] on the device."""
        if logits.shape[0] != len(rows):
            raise ValueError(f"{logits.shape[0]} logits rows but {len(rows)} sampling rows")
        if all(p.greedy for p, _, _ in rows):
            return ops.argmax(logits)
        packed = torch.from_numpy(pack_rows(rows).view(np.uint8).reshape(len(rows), 32))
        params = packed.pin_memory().to(self.device, non_blocking=True)
        return ops.sample(logits, params)

    def sample(self, logits: torch.Tensor, rows: Sequence[Tuple[SamplingParams, int, int]]) -> List[int]:
        ids = self.sample_device(logits, rows).cpu().tolist()
        if any(i < 0 for i in ids):
            raise RuntimeError("sampling produced no valid token for a row (were the logits finite?)")
        return ids
