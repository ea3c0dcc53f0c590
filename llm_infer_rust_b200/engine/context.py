"""What a part sees of one step: the batch's index arrays and its cache."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

import numpy as np
import torch


@dataclass
class StepContext:
    """One step's batch, as device int32 arrays (views of one buffer) plus host numbers.

    Rows are requests; a row of one token is a decode row, a longer row a
    portion of a prompt.  ``slots[g]`` and ``block_tables[g]`` belong to cache
    group ``g``.  ``host`` is the pinned host copy of the same buffer, for parts
    that need a number on the host; ``layout`` says where each array starts.
    """
    device: torch.device
    dtype: torch.dtype
    num_tokens: int
    num_rows: int
    num_decode: int
    num_prefill: int
    num_logits: int
    max_q_len: int
    max_kv_len: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    row_of_token: torch.Tensor
    cu_q: torch.Tensor
    kv_len: torch.Tensor
    prefix_len: torch.Tensor
    state_slots: torch.Tensor
    decode_rows: torch.Tensor
    prefill_rows: torch.Tensor
    logit_rows: torch.Tensor
    slots: List[torch.Tensor]
    block_tables: List[torch.Tensor]
    page_sizes: List[int]
    host: Optional[np.ndarray] = None
    layout: object = None
    # Upper bound of any row's length in this step (a replayed graph is built for the
    # longest sequence that may ever come, not for the one at capture).
    kv_len_bound: int = 0
    scratch: Optional[Callable[[int], torch.Tensor]] = None
    sm_count: int = 148
    extras: dict = field(default_factory=dict)


@dataclass
class LayerCache:
    """The cache of one entry of the run list."""
    group: int = -1                          # cache group of the pages, -1: no paged cache
    k: Optional[torch.Tensor] = None         # [pages + 1, page_size, kv_heads, head_dim]
    v: Optional[torch.Tensor] = None
    writes: bool = True                      # False: this entry reads another entry's pages
    state: Optional[torch.Tensor] = None     # [slots + 1, *state_shape]; slot 0 is the sink
