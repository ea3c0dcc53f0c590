"""Architecture-independent description of a decoder: pure data.

A ``ModelSpec`` says which parts make up every layer and in which order the
layers run.  It is produced by an architecture (from its typed configuration)
and consumed by the generic model builder, the cache planner and the weight
loader.  Nothing here knows a model family.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A configuration that the engine refuses, with the key and the reason."""


@dataclass(frozen=True)
class PartSpec:
    """One part: the name it is registered under and its sizes and constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """The parts of one layer, by name.  ``block`` names their arrangement and says which names it reads: the
    shipped ``pre_norm_deferred_add`` reads ``mixer``, ``feed_forward``, ``input_norm`` and ``post_mixer_norm``;
    an arrangement with other norm sites, four norms or two mixers reads other names, and nothing else changes."""
    block: PartSpec
    parts: Mapping[str, PartSpec]

    def __getitem__(self, name: str) -> PartSpec:
        try:
            return self.parts[name]
        except KeyError:
            raise ConfigError(f"the layer has no part named {name!r} (block {self.block.kind!r} asked for it); "
                              f"it has {sorted(self.parts)}") from None

    @staticmethod
    def pre_norm(block: PartSpec, mixer: PartSpec, feed_forward: PartSpec, input_norm: PartSpec,
                 post_mixer_norm: Optional[PartSpec] = None) -> "LayerSpec":
        """The usual decoder layer: a mixer and a feed-forward, each behind a norm (the same kind unless given)."""
        return LayerSpec(block, {"mixer": mixer, "feed_forward": feed_forward, "input_norm": input_norm,
                                 "post_mixer_norm": post_mixer_norm or input_norm})


@dataclass(frozen=True)
class RunEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers`` (the weights); the same layer may be
    named by several entries.  Every entry owns a cache of its own unless
    ``reads`` names an EARLIER entry of the run list: then this execution writes
    no keys and values and its mixer reads the cache of that entry.
    """
    layer: int
    reads: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    run_list: Tuple[RunEntry, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    position_encodings: Mapping[str, PartSpec] = field(default_factory=dict)

    def validate(self) -> None:
        for e, entry in enumerate(self.run_list):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"run list entry {e} names layer {entry.layer}, "
                                  f"the model has {len(self.layers)}")
            if entry.reads is not None:
                if not 0 <= entry.reads < e:
                    raise ConfigError(f"run list entry {e} reads the cache of entry {entry.reads}, "
                                      f"which does not run before it")
                if self.run_list[entry.reads].reads is not None:
                    raise ConfigError(f"run list entry {e} reads entry {entry.reads}, "
                                      f"which has no cache of its own")
