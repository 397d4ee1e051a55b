"""Random-weights mode: a model from a configuration and a seed.

Every element of every tensor is a function of (seed, the tensor's name, the
element's index in the stored tensor) alone, so the same seed gives the same
model whether it is drawn on the device straight into the engine's weight
buffer (``RandomSource``, csrc/randn_fill.cu) or on the host into a model
folder (``write_random_model``), and a tensor's values do not depend on which
other tensors exist:

    key   = mix64(seed * 0x9E3779B97F4A7C15 + fnv1a64(name))
    h     = mix64(key + (i + 1) * 0x9E3779B97F4A7C15)
    u1    = ((h >> 40) + 1) * 2^-24,  a = (h >> 8) & 0xFFFFFF
    z     = sqrt(-2 ln u1) * cos(2 pi a / 2^24)
    value = std * z                   (bfloat16: rounded to nearest even)

``ln`` and ``cos`` are fixed sequences of single 32-bit operations (below and,
operation for operation, in the kernel), which is what makes the two sides
agree to the bit.  Matrices are drawn with std ``matrix_std``, norm weights
with ``norm_std``.  The reference has no such mode (its tests hand-build
identity, zero and ramp tensors, src/engine/generate.rs:1477-1584).
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping, Tuple

import numpy as np
import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1

_M64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_CHUNK = 1 << 22          # elements drawn at a time on the host


def _mix64_int(z: int) -> int:
    z &= _M64
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & _M64
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return z


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of tensor ``name`` under ``seed``."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _M64
    return _mix64_int(((int(seed) & _M64) * _GOLDEN + h) & _M64)


def _mix64(z: np.ndarray) -> np.ndarray:
    z = z ^ (z >> np.uint64(30))
    z = z * np.uint64(0xBF58476D1CE4E5B9)
    z = z ^ (z >> np.uint64(27))
    z = z * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _f(x: float) -> np.float32:
    return np.float32(x)


def _ln_unit(u: np.ndarray) -> np.ndarray:
    bits = u.view(np.int32)
    e = (bits >> 23) - 127
    m = ((bits & 0x007FFFFF) | 0x3F800000).astype(np.int32).view(np.float32)
    big = m > _f(1.41421354)
    m = np.where(big, m * _f(0.5), m)
    e = np.where(big, e + 1, e)
    s = (m + _f(-1.0)) / (m + _f(1.0))
    s2 = s * s
    p = np.full_like(s, _f(0.111111111))
    for c in (0.142857143, 0.2, 0.333333333, 1.0):
        p = p * s2 + _f(c)
    return e.astype(np.float32) * _f(0.693147181) + (_f(2.0) * s) * p


def _cos_quarter(t: np.ndarray) -> np.ndarray:
    x = t * _f(1.57079633)
    x2 = x * x
    p = np.full_like(x, _f(-1.14707456e-11))
    for c in (2.08767570e-9, -2.75573192e-7, 2.48015873e-5, -1.38888889e-3, 4.16666667e-2,
              -0.5, 1.0):
        p = p * x2 + _f(c)
    return p


def _normals(key: int, first: int, count: int) -> np.ndarray:
    """z of elements first .. first + count - 1 as float32."""
    i = np.arange(first + 1, first + count + 1, dtype=np.uint64)
    h = _mix64(np.uint64(key) + i * np.uint64(_GOLDEN))
    u1 = ((h >> np.uint64(40)) + np.uint64(1)).astype(np.float32) * _f(2.0 ** -24)
    a = ((h >> np.uint64(8)) & np.uint64(0xFFFFFF)).astype(np.uint32)
    quadrant = a >> np.uint32(22)
    t = (a & np.uint32(0x3FFFFF)).astype(np.float32) * _f(2.0 ** -22)
    mirrored = (quadrant & np.uint32(1)) == 1
    c = _cos_quarter(np.where(mirrored, _f(1.0) + (-t), t))
    c = np.where((quadrant == 1) | (quadrant == 2), -c, c)
    r = np.sqrt(_f(-2.0) * _ln_unit(u1))
    return r * c


def randn_host_range(seed: int, name: str, std: float, first: int, count: int,
                     dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Elements ``first .. first + count - 1`` (in stored order) of tensor ``name``."""
    key = tensor_key(seed, name)
    out = np.empty(count, dtype=np.float32)
    with np.errstate(over="ignore"):
        for at in range(0, count, _CHUNK):
            n = min(_CHUNK, count - at)
            out[at:at + n] = _f(std) * _normals(key, first + at, n)
    return torch.from_numpy(out).to(dtype)


def randn_host(shape: Tuple[int, ...], seed: int, name: str, std: float,
               dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """The stored tensor ``name`` under ``seed`` on the host."""
    n = 1
    for s in shape:
        n *= int(s)
    return randn_host_range(seed, name, std, 0, n, dtype).view(tuple(shape))


def randn_device(shape: Tuple[int, ...], seed: int, name: str, std: float, dtype: torch.dtype,
                 device) -> torch.Tensor:
    """The same tensor drawn by the device's kernel (csrc/randn_fill.cu): the same bits."""
    from ..kernels import native
    rows = int(shape[0]) if len(shape) else 1
    cols = 1
    for s in shape[1:]:
        cols *= int(s)
    out = torch.empty(tuple(shape), dtype=dtype, device=device)
    native.randn_fill(out.view(1, rows, cols), rows, cols, 0, 0, tensor_key(seed, name), 0.0,
                      std, dtype)
    return out


def std_of(decl: TensorDecl, matrix_std: float, norm_std: float) -> float:
    return norm_std if decl.init == "norm" else matrix_std


def random_tensors(expected: Mapping[str, TensorDecl], seed: int, dtype: torch.dtype,
                   device="cpu", matrix_std: float = MATRIX_STD,
                   norm_std: float = NORM_STD) -> Dict[str, torch.Tensor]:
    """Every non-optional stored tensor of ``expected``, drawn in 32-bit and rounded once
    to ``dtype`` (bfloat16 or float32): on the host, or by the kernel when ``device`` is a
    CUDA device; both give the same bits."""
    device = torch.device(device)
    if dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"random weights are drawn as float32 or bfloat16, not {dtype}")
    out: Dict[str, torch.Tensor] = {}
    for name, decl in expected.items():
        if decl.optional:
            continue
        if decl.integer:
            out[name] = torch.zeros(decl.shape, dtype=torch.int32, device=device)
            continue
        std = std_of(decl, matrix_std, norm_std)
        if device.type == "cuda":
            out[name] = randn_device(tuple(decl.shape), seed, name, std, dtype, device)
        else:
            out[name] = randn_host(tuple(decl.shape), seed, name, std, dtype)
    return out


def write_random_model(model_dir: str, config: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16, matrix_std: float = MATRIX_STD,
                       norm_std: float = NORM_STD, device="cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a
    config.json dictionary) with seeded random weights; returns the folder.  ``device``:
    where the values are drawn (a CUDA device draws large models in seconds; the file is
    the same)."""
    from ..config.registry import spec_from_config
    from ..engine.model import expected_tensors
    _, spec = spec_from_config(config)
    tensors = random_tensors(expected_tensors(spec), seed, dtype, device, matrix_std, norm_std)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(dict(config), f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
