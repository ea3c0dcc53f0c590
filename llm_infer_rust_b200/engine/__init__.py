from ..cache import LayerCache
from .context import StepContext, context_from_layout
from .engine import Engine, GenerationResult, StepEntry, auto_chunked_prefill_size, graph_batch_sizes

__all__ = ["LayerCache", "StepContext", "context_from_layout", "Engine", "GenerationResult", "StepEntry",
           "auto_chunked_prefill_size", "graph_batch_sizes"]
