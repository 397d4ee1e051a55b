"""Token embedding and the output head.

Embedding: row gather, then a multiply by ``scale`` (the 32-bit residual
stream starts here).  Reference: src/model/layer.rs:1279-1288.

Head: the product of the (final-normed) wanted rows with the output matrix,
which is the embedding table when ``tied`` (src/engine/generate.rs:1106-1110),
then ``cap * tanh(logits / cap)`` when ``logit_softcap`` > 0.  Logits are
32-bit.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import native
from ..weights.arena import Piece, Resident
from ..weights.loader import TensorDecl
from .registry import register_embedding, register_head


class TokenEmbedding:
    captures_prompts = True   # row-wise: a recorded step of prompts may be replayed for others

    @staticmethod
    def tensors(params: Mapping, hidden: int, vocab: int) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((vocab, hidden))}

    @staticmethod
    def resident(params: Mapping, hidden: int, vocab: int) -> Dict[str, Resident]:
        return {"weight": Resident((vocab, hidden), pieces=(Piece("weight"),))}

    def __init__(self, params: Mapping, hidden: int, vocab: int,
                 weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.hidden = hidden
        self.vocab = vocab
        self.scale = float(params.get("scale", 1.0))
        self.table = rt.cast_matrix(weights["weight"])

    def forward(self, ctx) -> torch.Tensor:
        """The step's rows of the 32-bit residual stream.  An embedding gets the whole
        step context: one that adds learned positions reads ``ctx.row_pos`` too."""
        tokens = ctx.tokens
        h = torch.empty((tokens.numel(), self.hidden), dtype=torch.float32, device=tokens.device)
        return native.embed_rows(tokens, self.table, self.scale, h)


class LMHead:
    @staticmethod
    def tensors(params: Mapping, hidden: int, vocab: int) -> Dict[str, TensorDecl]:
        # a tied head uses the embedding's table; a file that stores the head's matrix
        # all the same is accepted and that tensor is not read
        return {"weight": TensorDecl((vocab, hidden), optional=bool(params.get("tied", True)))}

    @staticmethod
    def resident(params: Mapping, hidden: int, vocab: int) -> Dict[str, Resident]:
        if params.get("tied", True):
            return {}
        return {"weight": Resident((vocab, hidden), pieces=(Piece("weight"),))}

    def __init__(self, params: Mapping, hidden: int, vocab: int,
                 weights: Mapping[str, torch.Tensor], rt, embedding: Optional[TokenEmbedding]):
        self.rt = rt
        self.cap = float(params.get("logit_softcap") or 0.0)
        if params.get("tied", True):
            if embedding is None:
                raise ValueError("a tied head needs the embedding")
            self.weight = embedding.table
        else:
            self.weight = rt.cast_matrix(weights["weight"])

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        """y[n, hidden] in the activation type -> logits[n, vocab] in 32-bit."""
        epi = native.EPI_SOFTCAP if self.cap > 0 else native.EPI_NONE
        return self.rt.linear(y, self.weight, out_dtype=torch.float32, epilogue=epi, cap=self.cap)


register_embedding("token_embedding", TokenEmbedding)
register_head("lm_head", LMHead)
