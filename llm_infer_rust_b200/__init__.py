"""A single-GPU inference engine for B200 (sm_100a): dense Qwen3 first, built from
parts so that another architecture is a registry entry.

Public entry points:

* ``Engine(model_path, ...)`` with ``generate(prompts, sampling_params)`` and the
  step function ``step(entries)``;
* ``write_random_model(folder, config, seed)``: the random-weights mode;
* ``python -m llm_infer_rust_b200 --model-path DIR ...``: the command line;
* ``bin/trace_run``: trace replay.

Importing the package compiles nothing and needs no GPU; kernels are compiled
when an engine first needs them.
"""
from .config import (Architecture, ConfigError, ModelSpec, PartSpec, LayerSpec, RunEntry, Qwen3Config,
                     register_architecture, registered_architectures, resolve_architecture)
from . import architectures  # noqa: F401
from .sampling import SamplingParams
from .weights.random_init import random_tensors, write_random_model


def __getattr__(name):
    # The engine pulls in the CUDA side; keep `import llm_infer_rust_b200` light.
    if name in ("Engine", "StepEntry", "GenerationResult"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)


__all__ = ["Architecture", "ConfigError", "ModelSpec", "PartSpec", "LayerSpec", "RunEntry", "Qwen3Config",
           "register_architecture", "registered_architectures", "resolve_architecture", "SamplingParams",
           "random_tensors", "write_random_model", "Engine", "StepEntry", "GenerationResult"]
