from .base import BuildEnv, PagedKVSpec, ParamDecl, Part, StateSpec
from .registry import build_part, register_part, registered
from . import norm, position, feed_forward, embedding, attention, block  # noqa: F401  (registration)
from .model import DecoderModel

__all__ = ["BuildEnv", "PagedKVSpec", "ParamDecl", "Part", "StateSpec", "build_part", "register_part",
           "registered", "DecoderModel"]
