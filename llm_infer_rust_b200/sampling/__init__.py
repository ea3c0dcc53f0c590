from .sampler import ROW_DTYPE, Sampler, SamplingParams, pack_rows

__all__ = ["ROW_DTYPE", "Sampler", "SamplingParams", "pack_rows"]
