"""RMS norm: x * 1/sqrt(mean(x^2) + eps) * gain, statistics in 32-bit.

``unit_offset`` selects gain = 1 + weight (the convention of checkpoints
that store the weight as a deviation from one) instead of gain = weight
(the reference's convention, src/backend/cpu.rs:797-810, whose input files
already hold the effective gain).  The gain is formed once, in 32-bit, when
the weights are placed on the device.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import native
from ..weights.arena import Piece, Resident
from ..weights.loader import TensorDecl
from .registry import register_norm


class RMSNorm:
    fusable_rms = True

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((hidden,), init="norm")}

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        return {"gain": Resident((hidden,), torch.float32, (Piece("weight"),),
                                 1.0 if params.get("unit_offset", False) else 0.0)}

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.eps = float(params["eps"])
        self.hidden = hidden
        self.rt = rt
        self.gain = weights["gain"]

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.hidden), dtype=out_dtype or self.rt.dtype, device=x.device)
        return native.rms_norm(x, self.gain, self.eps, out, rows)


register_norm("rms_norm", RMSNorm)
