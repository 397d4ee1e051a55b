"""Architecture-neutral description of a decoder: what the engine builds from.

An architecture's typed configuration (read from its own ``config.json``
keys) is translated into a :class:`ModelSpec`.  From there on nothing knows
the architecture's name: the engine looks up each :class:`PartSpec`'s
``kind`` in the part registries (``parts/registry.py``) and hands it its
``params``.

The reference expresses the same choices as per-architecture default tuples
and per-layer flags inside one config struct (src/model/config.rs:59-123,
241-351, 379-385); here they are data, layer by layer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built; the message names the key."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered ``kind`` and its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: which block arrangement and which parts fill it.

    ``prefix`` is the common start of the layer's tensor names and ``names``
    gives, for each site of the block ("mixer", "feed_forward" and the norm
    sites), what follows it; a part only knows its own local names (such as
    ``q_proj.weight``) and never sees the whole name table.
    ``norms`` maps the block arrangement's norm sites to norm specs.
    """

    prefix: str
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec]
    names: Mapping[str, str]


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes :attr:`ModelSpec.layers` (the
    same index may appear more than once: the weights are then shared).
    ``cache_of`` names an earlier schedule entry whose keys and values (or
    state) this run reads instead of writing its own."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    names: Mapping[str, str] = field(default_factory=dict)  # "embedding", "final_norm", "head"
    stop_tokens: Tuple[int, ...] = ()

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0 or self.max_positions <= 0:
            raise ConfigError("hidden_size, vocab_size and max_positions must be positive")
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for pos, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule[{pos}] names layer {e.layer}, "
                                  f"but there are {len(self.layers)} layers")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < pos:
                    raise ConfigError(f"schedule[{pos}].cache_of={e.cache_of} must name "
                                      f"an earlier schedule entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule[{pos}].cache_of={e.cache_of} names an entry "
                                      f"that itself borrows a cache")


def require(d: Mapping[str, Any], key: str, typ=None) -> Any:
    """Fetch a required config.json key; the error names it."""
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if typ is int and (isinstance(v, bool) or not isinstance(v, int)):
        raise ConfigError(f"config.json: key '{key}' must be an integer, got {v!r}")
    if typ is float and (isinstance(v, bool) or not isinstance(v, (int, float))):
        raise ConfigError(f"config.json: key '{key}' must be a number, got {v!r}")
    return v
