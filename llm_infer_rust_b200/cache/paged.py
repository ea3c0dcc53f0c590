"""The paged cache: device tensors, their grouping and their sizing.

Host bookkeeping (which page holds what) lives in the C++ ``CacheManager``
(``csrc/host/page_cache.h``); this module decides the groups from the model,
sizes the pools and owns the tensors.

Grouping.  Every entry of the model's run list that keeps keys and values gets
tensors of its own, K and V of shape [pages + 1, kv_heads, page_size, head_dim]
(page 0 is the sink; the rows of one page and KV head are contiguous, so that the
copy engine fetches them as one block).  Entries whose mixers have the same NEED form a group: all
keys, or a window of W positions.  A group has its own page pool and every
request its own block table in it, so that a windowed group can give pages back
while the request runs.  Entries of one group may differ in head count and head
size: a page id indexes each entry's own tensors.  (The reference groups by
tensor geometry under one page-id space and has no windowed need:
src/engine/kvcache/spec.rs:7-18, src/engine/kvcache/pool.rs:128-228.)

Sizing follows the reference (src/engine/kvcache/allocator.rs:130-178):
budget = total * memory_ratio - used, pages = budget / bytes_per_page, with an
optional cap ``max_total_tokens`` (rounded down to whole pages).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..kernels.build import load_host_runtime


@dataclass
class LayerCache:
    """The cache of one entry of the run list."""
    group: int = -1                          # cache group of the pages, -1: no paged cache
    k: Optional[torch.Tensor] = None         # [pages + 1, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor] = None
    writes: bool = True                      # False: this entry reads another entry's pages
    state: Optional[torch.Tensor] = None     # [slots + 1, *state_shape]; slot 0 is the sink


@dataclass
class GroupPlan:
    window: Optional[int]
    page_size: int
    entries: List[int] = field(default_factory=list)     # run-list entries that own tensors here
    bytes_per_page: int = 0
    num_pages: int = 0


@dataclass
class CachePlan:
    groups: List[GroupPlan]
    group_of_entry: Dict[int, int]        # every run-list entry with a paged cache (owned or read)
    state_entries: Dict[int, object]      # run-list entry -> StateSpec


def plan_cache(model, page_size: int, itemsize: int) -> CachePlan:
    groups: List[GroupPlan] = []
    by_need: Dict[Optional[int], int] = {}
    group_of_entry: Dict[int, int] = {}
    state_entries: Dict[int, object] = {}
    for e, entry in enumerate(model.run_list):
        mixer = model.blocks[entry.layer].mixer
        state = mixer.state_spec()
        if state is not None:
            state_entries[e] = state
        kv = mixer.cache_spec()
        if kv is None:
            continue
        if entry.reads is not None:
            group_of_entry[e] = group_of_entry[entry.reads]
            continue
        need = kv.window
        if need not in by_need:
            by_need[need] = len(groups)
            groups.append(GroupPlan(need, page_size))
        g = by_need[need]
        groups[g].entries.append(e)
        groups[g].bytes_per_page += 2 * page_size * kv.num_kv_heads * kv.head_dim * itemsize
        group_of_entry[e] = g
    return CachePlan(groups, group_of_entry, state_entries)


def cache_budget_bytes(free: int, total: int, memory_ratio: float) -> int:
    """total * ratio - used, never more than what is free, never negative."""
    used = total - free
    return max(0, min(int(total * memory_ratio) - used, free))


def size_groups(plan: CachePlan, budget_bytes: Optional[int], max_total_tokens: Optional[int],
                max_requests: int, max_seq_len: int, max_step_tokens: int) -> None:
    """Fill ``num_pages`` of every group."""
    if not plan.groups:
        return
    P = plan.groups[0].page_size

    def window_cap(g: GroupPlan, pages_full: int) -> int:
        if g.window is None:
            return pages_full
        per_request = min(-(-max_seq_len // P), -(-(g.window + max_step_tokens - 1) // P) + 1)
        return min(pages_full, max_requests * per_request)

    if max_total_tokens is not None:
        pages = max_total_tokens // P
        if budget_bytes is not None:
            cost = sum(g.bytes_per_page for g in plan.groups)
            pages = min(pages, budget_bytes // max(cost, 1))
    else:
        if budget_bytes is None:
            raise ValueError("either a memory budget or max_total_tokens is needed to size the cache")
        # Largest `pages` such that sum_g bytes_per_page_g * cap_g(pages) fits the budget.
        lo, hi = 0, max(1, budget_bytes // max(min(g.bytes_per_page for g in plan.groups), 1))
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if sum(g.bytes_per_page * window_cap(g, mid) for g in plan.groups) <= budget_bytes:
                lo = mid
            else:
                hi = mid - 1
        pages = lo
    if pages < 1:
        raise MemoryError("the cache budget does not hold a single page beside the sink")
    for g in plan.groups:
        g.num_pages = window_cap(g, pages) if max_total_tokens is None else pages


class PagedCache:
    """Device tensors of the cache and the manager that books their pages."""

    def __init__(self, model, plan: CachePlan, max_requests: int, dtype: torch.dtype,
                 device: torch.device):
        rt = load_host_runtime()
        self.plan = plan
        self.dtype = dtype
        self.device = device
        self.page_sizes = [g.page_size for g in plan.groups]
        self.manager = rt.CacheManager(
            [rt.GroupSpec(g.page_size, g.num_pages, g.window or 0) for g in plan.groups], max_requests)
        owned: Dict[int, LayerCache] = {}
        self.layer_caches: List[LayerCache] = []
        for e, entry in enumerate(model.run_list):
            mixer = model.blocks[entry.layer].mixer
            cache = LayerCache()
            kv = mixer.cache_spec()
            if kv is not None:
                g = plan.group_of_entry[e]
                cache.group = g
                if entry.reads is None:
                    shape = (plan.groups[g].num_pages + 1, kv.num_kv_heads, plan.groups[g].page_size, kv.head_dim)
                    cache.k = torch.zeros(shape, dtype=dtype, device=device)
                    cache.v = torch.zeros(shape, dtype=dtype, device=device)
                    owned[e] = cache
                else:
                    cache.k, cache.v, cache.writes = owned[entry.reads].k, owned[entry.reads].v, False
            state = plan.state_entries.get(e)
            if state is not None:
                cache.state = torch.zeros((max_requests + 1,) + tuple(state.shape), dtype=state.dtype,
                                          device=device)
            self.layer_caches.append(cache)

    def bytes(self) -> int:
        total = 0
        for c in self.layer_caches:
            if c.writes and c.k is not None:
                total += 2 * c.k.numel() * c.k.element_size()
            if c.state is not None:
                total += c.state.numel() * c.state.element_size()
        return total
