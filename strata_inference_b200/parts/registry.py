"""Registries of parts by ``kind``.

``register_mixer("my_kind", MyMixer)`` makes ``PartSpec("my_kind", {...})``
buildable anywhere a mixer is expected; the same holds for feed-forwards,
norms, position encodings, blocks, embeddings and heads.  The built-in
parts register themselves when ``strata_inference_b200.parts`` is imported.
"""

from __future__ import annotations

from typing import Callable, Dict

from ..config.spec import ConfigError, PartSpec

_REGISTRIES: Dict[str, Dict[str, type]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {},
    "block": {}, "embedding": {}, "head": {},
}


def _register(role: str, kind: str, cls: type) -> type:
    _REGISTRIES[role][kind] = cls
    return cls


def register_mixer(kind: str, cls: type) -> type:
    return _register("mixer", kind, cls)


def register_feed_forward(kind: str, cls: type) -> type:
    return _register("feed_forward", kind, cls)


def register_norm(kind: str, cls: type) -> type:
    return _register("norm", kind, cls)


def register_position(kind: str, cls: type) -> type:
    return _register("position", kind, cls)


def register_block(kind: str, cls: type) -> type:
    return _register("block", kind, cls)


def register_embedding(kind: str, cls: type) -> type:
    return _register("embedding", kind, cls)


def register_head(kind: str, cls: type) -> type:
    return _register("head", kind, cls)


def part_class(role: str, kind: str) -> type:
    table = _REGISTRIES[role]
    if kind not in table:
        raise ConfigError(f"no {role} of kind '{kind}' is registered; "
                          f"known: {', '.join(sorted(table)) or '(none)'}")
    return table[kind]


def known(role: str):
    return tuple(sorted(_REGISTRIES[role]))
