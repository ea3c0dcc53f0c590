from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import (Architecture, register_architecture, registered_architectures,
                       resolve_architecture)
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Architecture",
           "register_architecture", "registered_architectures", "resolve_architecture",
           "Qwen3Config"]
