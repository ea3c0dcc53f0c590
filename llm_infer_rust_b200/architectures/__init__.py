"""Importing this package registers the architectures that ship with the engine."""
from . import qwen3  # noqa: F401
