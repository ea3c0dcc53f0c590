from .paged import CachePlan, GroupPlan, LayerCache, PagedCache, cache_budget_bytes, plan_cache, size_groups

__all__ = ["CachePlan", "GroupPlan", "LayerCache", "PagedCache", "cache_budget_bytes", "plan_cache", "size_groups"]
