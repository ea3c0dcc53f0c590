from .context import LayerCache, StepContext
from .engine import Engine, GenerationResult, StepEntry, auto_chunked_prefill_size, graph_batch_sizes

__all__ = ["LayerCache", "StepContext", "Engine", "GenerationResult", "StepEntry",
           "auto_chunked_prefill_size", "graph_batch_sizes"]
