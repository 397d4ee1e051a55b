"""Checked loading: the file's table of tensors against the model's.

The model's parts declare which tensors they need (name, shape); this module
compares that table with what a model folder holds and raises ONE error that
lists everything wrong: tensors that are missing, tensors nobody asked for,
and tensors of the wrong shape or kind.  The reference reports the first
missing tensor only (src/model/weights.rs:133-193, src/error.rs:32).

Storage types are kept: bfloat16 stays bfloat16, a tensor stored in 32-bit
stays in 32-bit, float16 (which no kernel here computes in) becomes
bfloat16, integer tables become int32.  Parts cast what they feed to matrix
products to the engine's compute type when they are built.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from .safetensors_io import ModelFiles


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part needs.  ``init`` tells the random-weights mode how to
    fill it: "matrix" (projection and embedding matrices) or "norm" (norm
    weights); ``integer`` marks index tables."""

    shape: Tuple[int, ...]
    init: str = "matrix"
    optional: bool = False
    integer: bool = False


class WeightError(ValueError):
    """What is wrong with a model folder's tensors, all of it at once."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_kind: List[Tuple[str, str]]):
        self.missing = missing
        self.unexpected = unexpected
        self.wrong_shape = wrong_shape
        self.wrong_kind = wrong_kind
        lines = [f"{where}: the tensors do not fit the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        if wrong_kind:
            lines.append(f"  wrong type ({len(wrong_kind)}): " + ", ".join(
                f"{n} {why}" for n, why in wrong_kind))
        super().__init__("\n".join(lines))


def check_table(where: str, have: Mapping[str, Tuple[Tuple[int, ...], torch.dtype]],
                expected: Mapping[str, TensorDecl]) -> None:
    """Raise :class:`WeightError` unless ``have`` is exactly what ``expected`` needs."""
    missing = [n for n, d in expected.items() if n not in have and not d.optional]
    unexpected = [n for n in have if n not in expected]
    wrong_shape, wrong_kind = [], []
    for n, d in expected.items():
        if n not in have:
            continue
        shape, dtype = have[n]
        if tuple(shape) != tuple(d.shape):
            wrong_shape.append((n, tuple(shape), tuple(d.shape)))
        if d.integer and dtype.is_floating_point:
            wrong_kind.append((n, f"is stored as {dtype}, expected an integer table"))
        if not d.integer and not dtype.is_floating_point:
            wrong_kind.append((n, f"is stored as {dtype}, expected floating point"))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightError(where, sorted(missing), sorted(unexpected), wrong_shape, wrong_kind)


def storage_dtype(stored: torch.dtype) -> torch.dtype:
    """The type a stored tensor is kept in."""
    if not stored.is_floating_point:
        return torch.int32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_weights(model_dir: str, expected: Mapping[str, TensorDecl],
                 device: torch.device) -> Dict[str, torch.Tensor]:
    """Read every expected tensor of ``model_dir`` onto ``device``."""
    files = ModelFiles(model_dir)
    have = {n: (files.shape(n), files.dtype(n)) for n in files.names()}
    check_table(model_dir, have, expected)
    out: Dict[str, torch.Tensor] = {}
    for n in expected:
        if n not in have:
            continue
        t = files.get(n)
        out[n] = t.to(device=device, dtype=storage_dtype(t.dtype))
    return out
