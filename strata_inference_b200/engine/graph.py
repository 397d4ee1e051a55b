"""Single-token steps replayed from a CUDA graph.

Decoding launches a few hundred small kernels per step; launched one by one
from the host they cost more than they run.  A :class:`DecodeGraph` captures
the kernel sequence of one single-token step plus sampling for a fixed
number of sequences and replays it: what changes between steps (tokens,
positions, slots, page tables, generator states) lives in device buffers at
fixed addresses that are refreshed before each replay, and no launch shape
depends on the sequences' lengths.  The kernels are the ones ``Engine.step``
launches.
"""

from __future__ import annotations

import gc
from typing import Optional, Sequence

import torch

from ..kernels import native
from ..parts.base import StepContext


_STAGES = 4      # steps a caller may be ahead of the device


class DecodeGraph:
    def __init__(self, engine, n_seqs: int, temperature: float, top_k: int, top_p: float):
        self.engine = engine
        self.B = B = n_seqs
        self.temperature, self.top_k, self.top_p = temperature, top_k, top_p
        # Pinned staging buffers for the metadata, used in turn: a caller may issue steps
        # without waiting for them, and a buffer must not be rewritten before its copy ran.
        self.hosts = [torch.zeros(8 * B, dtype=torch.int32).pin_memory() for _ in range(_STAGES)]
        self.copied = [None] * _STAGES
        ar = torch.arange(B, dtype=torch.int32)
        for host in self.hosts:
            for field in (2, 6, 7):      # row_seq, seq_row0, wanted rows: 0..B-1
                host[field * B:(field + 1) * B] = ar
        self.meta = torch.zeros(8 * B, dtype=torch.int32, device=engine.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out: Optional[torch.Tensor] = None
        self.logits: Optional[torch.Tensor] = None
        self.last_logits: Optional[torch.Tensor] = None
        self.calls = 0
        self.launches_per_step = 0

    def _field(self, i: int) -> torch.Tensor:
        return self.meta[i * self.B:(i + 1) * self.B]

    def _forward(self, slots, starts):
        eng, B = self.engine, self.B
        ctx = StepContext(
            n_rows=B, n_seqs=B, tokens=self._field(0), row_pos=self._field(1),
            row_seq=self._field(2), seq_slot=self._field(3), seq_start=self._field(4),
            seq_end=self._field(5), seq_row0=self._field(6), starts=list(starts),
            counts=[1] * B, slots=list(slots), all_from_start=False, max_count=1,
            max_end=max(starts) + 1, cache=eng.cache, runtime=eng.rt, graph_capture=True)
        h = eng.model.hidden_states(ctx)
        logits = eng.model.logits(h, self._field(7))
        out = torch.empty(B, dtype=torch.int32, device=eng.device)
        native.sample_rows(logits, self.temperature, self.top_k, self.top_p, eng.rng_state, out,
                           self._field(3))
        return logits, out

    def run(self, slots: Sequence[int], tokens: Sequence[int], use_graph: bool = True):
        eng, B = self.engine, self.B
        if len(slots) != B or len(tokens) != B:
            raise ValueError(f"this graph steps {B} sequences")
        V = eng.vocab_size
        for t in tokens:
            if not 0 <= int(t) < V:
                raise ValueError(f"input token ID {t} exceeds vocab_size {V}")
        slots = [int(s) for s in slots]
        eng.cache.reserve([(s, 1) for s in slots])
        starts = [eng.cache.length(s) for s in slots]
        stage = self.calls % _STAGES
        if self.copied[stage] is not None:
            self.copied[stage].synchronize()     # (long done unless the caller runs far ahead)
        h = self.hosts[stage]
        h[0:B] = torch.tensor([int(t) for t in tokens], dtype=torch.int32)
        st = torch.tensor(starts, dtype=torch.int32)
        h[B:2 * B] = st
        h[3 * B:4 * B] = torch.tensor(slots, dtype=torch.int32)
        h[4 * B:5 * B] = st
        h[5 * B:6 * B] = st + 1
        self.meta.copy_(h, non_blocking=True)
        if self.copied[stage] is None:
            self.copied[stage] = torch.cuda.Event()
        self.copied[stage].record()
        eng.cache.sync_tables()
        if self.graph is not None and use_graph:
            self.graph.replay()
            result, self.last_logits = self.out, self.logits
        else:
            before = native.launch_count()
            self.last_logits, result = self._forward(slots, starts)
            self.launches_per_step = native.launch_count() - before
            if use_graph and self.calls >= 1:
                # The eager run above was this step (and warmed up every library
                # the step uses).  The capture records the same launches for the
                # steps to come and runs nothing; its output buffers are the ones
                # later replays fill.
                # Nothing but the step's own launches may touch CUDA while it is recorded.  The
                # garbage collector could: when it frees a pinned buffer of an engine that
                # is gone, the host allocator asks CUDA about that buffer's events, which
                # invalidates a capture in progress.  So it collects before and stays off
                # until the capture has ended.
                g = torch.cuda.CUDAGraph()
                collecting = gc.isenabled()
                gc.collect()
                gc.disable()
                try:
                    with torch.cuda.graph(g, capture_error_mode="thread_local"):
                        self.logits, self.out = self._forward(slots, starts)
                finally:
                    if collecting:
                        gc.enable()
                self.graph = g
        self.calls += 1
        for s in slots:
            eng.cache.advance(s, 1)
        return result
