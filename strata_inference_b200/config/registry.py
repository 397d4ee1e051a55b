"""One table from an architecture's name to its configuration and model spec.

The reference selects the architecture with a ``match`` on the name string
and a tuple of per-architecture defaults (src/model/config.rs:136-150,
241-351).  Here an architecture is one row: a function that parses
``config.json`` into its typed configuration and a function that lays that
configuration out as a :class:`~.spec.ModelSpec`.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Tuple

from .spec import ConfigError, ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(names, parse_config, build_spec) -> None:
    """Add a row.  ``names`` are the strings config.json may carry in
    ``architectures`` or ``model_type``."""
    if isinstance(names, str):
        names = (names,)
    arch = Architecture(names[0], parse_config, build_spec)
    for n in names:
        _ARCHITECTURES[n] = arch


def known_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(config: Mapping[str, Any]) -> Architecture:
    """Find the row for a config.json dictionary."""
    names = list(config.get("architectures") or [])
    if config.get("model_type"):
        names.append(config["model_type"])
    if not names:
        raise ConfigError("config.json: neither 'architectures' nor 'model_type' is given; "
                          f"known architectures: {', '.join(known_architectures())}")
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    raise ConfigError(f"unsupported architecture {', '.join(map(repr, names))}; "
                      f"known architectures: {', '.join(known_architectures())}")


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file")
    with open(path) as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None


def spec_from_config(config: Mapping[str, Any]) -> Tuple[Any, ModelSpec]:
    """config.json dictionary -> (typed configuration, model spec)."""
    arch = architecture_of(config)
    typed = arch.parse_config(config)
    return typed, arch.build_spec(typed)


def _register_builtin() -> None:
    from .gemma2 import Gemma2Config, gemma2_spec
    register_architecture(("Gemma2ForCausalLM", "gemma2"), Gemma2Config.from_dict, gemma2_spec)


_register_builtin()
