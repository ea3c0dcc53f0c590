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


def context_from_layout(layout, dev: torch.Tensor, host: Optional[torch.Tensor], page_sizes: List[int],
                        device: torch.device, dtype: torch.dtype, kv_len_bound: int,
                        scratch: Optional[Callable[[int], torch.Tensor]] = None,
                        sm_count: int = 148) -> StepContext:
    """Views of the device buffer ``dev`` that the batch builder's ``layout`` describes."""
    def view(off, n):
        return dev[off:off + n]

    groups = len(page_sizes)
    T, R = layout.num_tokens, layout.num_rows
    return StepContext(
        device=device, dtype=dtype, num_tokens=T, num_rows=R, num_decode=layout.num_decode,
        num_prefill=layout.num_prefill, num_logits=layout.num_logits, max_q_len=layout.max_q_len,
        max_kv_len=layout.max_kv_len,
        token_ids=view(layout.off_tokens, T), positions=view(layout.off_positions, T),
        row_of_token=view(layout.off_row_of_token, T), cu_q=view(layout.off_cu_q, R + 1),
        kv_len=view(layout.off_kv_len, R), prefix_len=view(layout.off_prefix_len, R),
        state_slots=view(layout.off_state_slot, R),
        decode_rows=view(layout.off_decode_rows, layout.num_decode),
        prefill_rows=view(layout.off_prefill_rows, layout.num_prefill),
        logit_rows=view(layout.off_logit_rows, layout.num_logits),
        slots=[view(layout.off_slots[g], T) for g in range(groups)],
        block_tables=[view(layout.off_table[g], R * layout.table_width[g]).view(R, layout.table_width[g])
                      for g in range(groups)],
        page_sizes=list(page_sizes),
        host=None if host is None else host.numpy(), layout=layout, kv_len_bound=kv_len_bound,
        scratch=scratch, sm_count=sm_count)
