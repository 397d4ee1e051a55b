"""Position encodings of the attention mixer.

``rope_neox``: rotary embedding with half-split pairs (x[i], x[i + rot/2]);
``rope_interleaved``: pairs (x[2i], x[2i+1]).  Frequencies follow the
reference: freq_i = theta^((-1/rot) * 2i) evaluated in 32-bit
(src/backend/cpu.rs:1276-1282); the angle pos * freq_i and its sine and
cosine are taken in 32-bit inside the kernel (csrc/rope_cache.cu).
``none``: no encoding.

A position part offers ``rotary()`` -> (inv_freq, rotary_dim, style) for the
fused rotate-and-store kernel.  A part without ``rotary`` must offer
``apply(q, k, ctx)`` instead, which rotates the ``[rows, heads, head_dim]``
views in place before keys are stored.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional, Tuple

import torch

from ..config.spec import ConfigError
from ..kernels import native
from ..weights.loader import TensorDecl
from .registry import register_position


class Rope:
    style = native.ROPE_HALF_SPLIT

    @staticmethod
    def tensors(params: Mapping, head_dim: int) -> Dict[str, TensorDecl]:
        return {}

    def __init__(self, params: Mapping, head_dim: int, weights: Mapping[str, torch.Tensor], rt):
        self.theta = float(params["theta"])
        self.rotary_dim = int(params.get("rotary_dim") or head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ConfigError(f"rotary_dim {self.rotary_dim} must be even and at most "
                              f"head_dim {head_dim}")
        inv_ndims = torch.tensor(-1.0 / self.rotary_dim, dtype=torch.float32)
        two_i = torch.arange(self.rotary_dim // 2, dtype=torch.float32) * 2.0
        freqs = torch.pow(torch.tensor(self.theta, dtype=torch.float32), inv_ndims * two_i)
        self.inv_freq = freqs.to(rt.device).contiguous()

    def rotary(self) -> Tuple[Optional[torch.Tensor], int, int]:
        return self.inv_freq, self.rotary_dim, self.style


class RopeInterleaved(Rope):
    style = native.ROPE_INTERLEAVED


class NoPosition:
    @staticmethod
    def tensors(params: Mapping, head_dim: int) -> Dict[str, TensorDecl]:
        return {}

    def __init__(self, params: Mapping, head_dim: int, weights, rt):
        pass

    def rotary(self):
        return None, 0, native.ROPE_HALF_SPLIT


register_position("rope_neox", Rope)
register_position("rope_interleaved", RopeInterleaved)
register_position("none", NoPosition)
