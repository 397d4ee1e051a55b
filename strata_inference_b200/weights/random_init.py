"""Random-weights mode: a model folder from a configuration and a seed.

Matrices are drawn from N(0, matrix_std) and norm weights from
N(0, norm_std); every tensor has its own generator keyed by (seed, name), so
a tensor's values do not depend on which other tensors exist.  The
reference has no such mode (its tests hand-build identity, zero and ramp
tensors, src/engine/generate.rs:1477-1584).
"""

from __future__ import annotations

import json
import os
import zlib
from typing import Any, Dict, Mapping, Optional

import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _generator(seed: int, name: str, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensors(expected: Mapping[str, TensorDecl], seed: int, dtype: torch.dtype,
                   device="cpu", matrix_std: float = MATRIX_STD,
                   norm_std: float = NORM_STD) -> Dict[str, torch.Tensor]:
    """Draw every non-optional tensor of ``expected``.  Values are drawn in
    32-bit and rounded once to ``dtype``."""
    device = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    for name, decl in expected.items():
        if decl.optional:
            continue
        g = _generator(seed, name, device)
        if decl.integer:
            out[name] = torch.zeros(decl.shape, dtype=torch.int32, device=device)
            continue
        std = norm_std if decl.init == "norm" else matrix_std
        t = torch.empty(decl.shape, dtype=torch.float32, device=device)
        t.normal_(0.0, std, generator=g)
        out[name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, config: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16, matrix_std: float = MATRIX_STD,
                       norm_std: float = NORM_STD) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a
    config.json dictionary) with seeded random weights; returns the folder."""
    from ..config.registry import spec_from_config
    from ..engine.model import expected_tensors
    _, spec = spec_from_config(config)
    tensors = random_tensors(expected_tensors(spec), seed, dtype, "cpu", matrix_std, norm_std)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(dict(config), f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
