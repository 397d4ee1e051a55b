"""What every part is built with and what it is stepped with.

A *part* (mixer, feed-forward, norm, position encoding, block, embedding,
head) is a class registered under a ``kind`` name in ``parts/registry.py``.
It gets its sizes and constants as ``params`` (from a PartSpec), the hidden
size, its own tensors under their local names, and a :class:`Runtime`.  It
never learns which model it is in.

Interfaces (duck-typed; the toy parts of the tests implement exactly these):

``Mixer``
    ``tensors(params, hidden) -> {local name: TensorDecl}`` (static),
    ``cache_need() -> CacheNeed | None``,
    ``forward(x, ctx, entry, cache_entry, owns_cache) -> y`` with x, y
    ``[rows, hidden]`` in the activation type.  ``entry`` is the schedule
    position being run, ``cache_entry`` the schedule position whose cache it
    uses (the same unless the schedule lends it another's), ``owns_cache``
    whether it may write there.
``FeedForward``
    ``tensors(params, hidden)``, ``forward(x, ctx) -> y``.
``Norm``
    ``tensors(params, hidden)``, ``forward(x, out_dtype, rows=None) -> y``
    (x 32-bit or activation type; ``rows`` selects rows of x).  A norm that
    also has ``gain`` (32-bit ``[hidden]``) and ``eps`` and sets
    ``fusable_rms = True`` can be fused by blocks into the residual kernel.
``Position``
    ``tensors(params, head_dim)`` (usually none); either ``rotary()`` returning
    ``(inv_freq, rotary_dim, style)`` for the fused rotate-and-store kernel, or
    ``apply(q, k, ctx)`` rotating ``[rows, heads, head_dim]`` views in place.
``Block``
    ``forward(h, normed, ctx, entry, cache_entry, owns_cache, next_norm)``:
    ``h`` is the 32-bit residual stream, updated in place; ``normed`` is
    ``first_norm(h)`` if the previous block already made it; the block returns
    ``next_norm(h)`` when it can fuse that, else ``None``.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..cache.paged import KVView, SequenceCache
from ..kernels import native


class Runtime:
    """Device, compute type and the matrix product, shared by all parts."""

    def __init__(self, device, dtype: torch.dtype):
        self.device = torch.device(device)
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute type must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        native.require_device(self.device)
        native.library()
        # true 32-bit products: no reduced-precision matrix mode anywhere
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")
        # Up to this many rows a product goes to the weight-streaming kernel (which
        # takes up to native.SKINNY_MAX_ROWS); measured on a B200 at Gemma2-2B sizes it
        # is ahead of the library product up to 16 rows and behind it from 32 on.
        self.skinny_max_rows = 16
        # SIB_FUSE_ROTATION=0: rotation and cache write always run as a kernel of their own
        self.fuse_rotation = os.environ.get("SIB_FUSE_ROTATION", "1") != "0"
        # from this many rows on the gate/up product with its gated epilogue (pairs of SMs,
        # 256 x 256 tiles) beats the library product followed by the activation kernel
        self.gated_gemm_min_rows = 128
        self._scratch: Optional[torch.Tensor] = None
        self._tickets: Optional[torch.Tensor] = None
        self._retired: list = []       # outgrown buffers that captured graphs may still name

    def cast_matrix(self, w: torch.Tensor) -> torch.Tensor:
        """A weight matrix in the compute type, contiguous, on the device."""
        return w.to(device=self.device, dtype=self.dtype).contiguous()

    def scratch(self, n_bytes: int) -> torch.Tensor:
        """A persistent scratch buffer of at least ``n_bytes``.  It grows by doubling; a buffer
        that was outgrown is kept, because a captured graph may still write into it."""
        if self._scratch is None or self._scratch.numel() < n_bytes:
            have = self._scratch.numel() if self._scratch is not None else 0
            self._retired.append(self._scratch)
            self._scratch = torch.empty(max(n_bytes, 2 * have, 1 << 20), dtype=torch.uint8,
                                        device=self.device)
        return self._scratch

    def tickets(self, n: int) -> torch.Tensor:
        """At least ``n`` int32 counters that are zero whenever no kernel is
        running: kernels that count their blocks through them put them back."""
        if self._tickets is None or self._tickets.numel() < n:
            self._retired.append(self._tickets)
            self._tickets = torch.zeros(max(n, 4096), dtype=torch.int32, device=self.device)
        return self._tickets

    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
               epilogue: int = native.EPI_NONE, cap: float = 0.0) -> torch.Tensor:
        """x[R, K] . w[N, K]^T.  Few bfloat16 rows go to the weight-streaming
        kernel of this package; everything else is a library matrix product
        (cuBLAS through torch, in the operands' own precision), as in the
        reference, which calls cuBLAS for every product
        (src/backend/cuda/mod.rs:828-905)."""
        out_dtype = out_dtype or x.dtype
        R, K = x.shape
        N = w.shape[0]
        n_out = N // 2 if epilogue == native.EPI_GEGLU else N
        if (x.dtype == torch.bfloat16 and 0 < R <= self.skinny_max_rows and K % 8 == 0
                and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0):
            out = torch.empty((R, n_out), dtype=out_dtype, device=x.device)
            return native.skinny_linear(x, w, out, epilogue, cap)
        aligned = (K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                   and x.data_ptr() % 16 == 0)
        fused_gate = epilogue == native.EPI_GEGLU and R > self.gated_gemm_min_rows
        if x.dtype == torch.bfloat16 and aligned and (out_dtype == torch.float32 or fused_gate):
            # the tcgen05 product where its epilogue saves a pass over the outputs: 32-bit
            # logits of many rows, soft-capped as they are written; the gated activation of
            # the feed-forward, which halves what is written and spares a second kernel
            out = torch.empty((R, n_out), dtype=out_dtype, device=x.device)
            return native.gemm_tcgen05(x, w, out, epilogue, cap)
        if epilogue == native.EPI_GEGLU:
            raise ValueError("the gated epilogue exists in the hand-written products only")
        if out_dtype == x.dtype:
            y = torch.matmul(x, w.t())
        else:
            y = torch.mm(x, w.t(), out_dtype=out_dtype)
        if epilogue == native.EPI_SOFTCAP:
            if y.dtype != torch.float32:
                raise ValueError("the soft cap epilogue is applied to 32-bit outputs")
            native.softcap_(y, cap)
        return y


@dataclass
class StepContext:
    """One step's rows: which sequence and position each row is, on the
    device for the kernels and on the host for launch decisions."""

    n_rows: int
    n_seqs: int
    tokens: torch.Tensor      # [rows] int32
    row_pos: torch.Tensor     # [rows] absolute position of the row
    row_seq: torch.Tensor     # [rows] index of the row's sequence in this step
    seq_slot: torch.Tensor    # [seqs] cache slot
    seq_start: torch.Tensor   # [seqs] length before the step
    seq_end: torch.Tensor     # [seqs] length after the step
    seq_row0: torch.Tensor    # [seqs] packed index of the sequence's first row
    starts: List[int]         # host copies
    counts: List[int]
    slots: List[int]
    all_from_start: bool      # every sequence begins at position 0 in this step
    max_count: int
    max_end: int
    cache: SequenceCache
    runtime: Runtime
    graph_capture: bool = False   # the step is being captured into a CUDA graph: launch shapes must not depend on lengths

    def kv(self, entry: int) -> KVView:
        return self.cache.kv_view(entry)

    def state(self, entry: int) -> torch.Tensor:
        return self.cache.state_view(entry)
