"""The dense gated feed-forward: down(act(gate(x)) * up(x)), no biases.

Reference: src/model/layer.rs:696-710 (two products, the gated activation,
the down product), src/backend/cpu.rs:1190-1199 (tanh-GELU).  The gate and up
matrices are kept as ONE matrix so that one product makes both halves; when
the intermediate size allows it their rows are interleaved in groups of 8
(8 gate rows, then the 8 matching up rows), which puts a gate value and its
up value into the same thread of the weight-streaming kernel, whose epilogue
then writes act(gate) * up directly.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config.spec import ConfigError
from ..kernels import native
from ..weights.arena import Piece, Resident
from ..weights.loader import TensorDecl
from .registry import register_feed_forward

_ACTIVATIONS = ("gelu_pytorch_tanh",)
_GROUP = 8


class GatedMLP:
    chain_safe = True      # deferred results are read by this runtime's and native's launchers only
    captures_prompts = True   # row-wise: a recorded step of prompts may be replayed for others

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        inter = params["intermediate_size"]
        return {
            "gate_proj.weight": TensorDecl((inter, hidden)),
            "up_proj.weight": TensorDecl((inter, hidden)),
            "down_proj.weight": TensorDecl((hidden, inter)),
        }

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        """Gate and up as ONE matrix: runs of 8 gate rows followed by the 8 matching up
        rows when the intermediate size is a multiple of 8, else all gates, then all ups."""
        inter = int(params["intermediate_size"])
        if inter % _GROUP == 0:
            pieces = (Piece("gate_proj.weight", 0, _GROUP, 2 * _GROUP),
                      Piece("up_proj.weight", _GROUP, _GROUP, 2 * _GROUP))
        else:
            pieces = (Piece("gate_proj.weight", 0), Piece("up_proj.weight", inter))
        return {
            "gate_up_proj.weight": Resident((2 * inter, hidden), pieces=pieces),
            "down_proj.weight": Resident((hidden, inter), pieces=(Piece("down_proj.weight"),)),
        }

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.inter = int(params["intermediate_size"])
        act = params.get("activation", _ACTIVATIONS[0])
        if act not in _ACTIVATIONS:
            raise ConfigError(f"gated_mlp: activation {act!r} is not supported; "
                              f"known: {', '.join(_ACTIVATIONS)}")
        self.group = _GROUP if self.inter % _GROUP == 0 else 0
        self.w_gate_up = rt.cast_matrix(weights["gate_up_proj.weight"])
        self.w_down = rt.cast_matrix(weights["down_proj.weight"])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        rt = self.rt
        R = x.shape[0]
        if (self.group == _GROUP and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                and (R <= rt.skinny_max_rows or R > rt.gated_gemm_min_rows
                     or (rt.chain is not None and R <= rt.chain_max_rows))):
            t = rt.linear(x, self.w_gate_up, epilogue=native.EPI_GEGLU)
        else:
            gate_up = rt.linear(x, self.w_gate_up)
            t = torch.empty((R, self.inter), dtype=x.dtype, device=x.device)
            native.gelu_mul(gate_up, t, self.group)
        return rt.linear(t, self.w_down)


register_feed_forward("gated_mlp", GatedMLP)
