"""Steps replayed from CUDA graphs: single-token steps, and short prompt steps.

Decoding launches a few hundred small kernels per step; launched one by one
from the host they cost more than they run.  A :class:`DecodeGraph` captures
the kernel sequence of one single-token step plus sampling for a fixed
number of sequences and replays it: what changes between steps (tokens,
positions, slots, page tables, generator states) lives in device buffers at
fixed addresses that are refreshed before each replay, and no launch shape
depends on the sequences' lengths.  The kernels are the ones ``Engine.step``
launches.

A :class:`PromptGraph` does the same for a step of prompts that all start at position 0
and have few enough rows that launching them from the host costs more than running them:
it is recorded for a number of sequences, a number of wanted rows and a number of rows
rounded up, and a replay fills the rows that are left over with a sequence that holds no
slot, whose keys and values are not stored.  No other row's result depends on those rows.
"""

from __future__ import annotations

import gc
from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import native
from ..parts.base import StepContext


_STAGES = 4      # steps a caller may be ahead of the device


class DecodeGraph:
    def __init__(self, engine, n_seqs: int, temperature: float, top_k: int, top_p: float,
                 span: Optional[int] = None):
        self.engine = engine
        self.B = B = n_seqs
        self.span = span      # the attention's work is divided for sequences of up to this length
        self.temperature, self.top_k, self.top_p = temperature, top_k, top_p
        # Pinned staging buffers for the step's integers, used in turn: a caller may issue
        # steps without waiting for them, and a buffer must not be rewritten before its
        # copy ran.
        size = StepContext.packed_size(B, B, B)
        self.hosts = [torch.zeros(size, dtype=torch.int32).pin_memory() for _ in range(_STAGES)]
        self.host_rows = [h.numpy().reshape(8, B) for h in self.hosts]     # views of the same memory
        self.copied = [None] * _STAGES
        self.meta = torch.zeros(size, dtype=torch.int32, device=engine.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out: Optional[torch.Tensor] = None
        self.logits: Optional[torch.Tensor] = None
        self.last_logits: Optional[torch.Tensor] = None
        self.calls = 0
        self.launches_per_step = 0
        self.last_slots: Optional[list] = None      # of the latest run
        self.out_is_latest = False      # whether `out` holds the tokens that the latest run sampled

    def _forward(self, seqs, capture: bool):
        eng, B = self.engine, self.B
        ctx = StepContext(self.meta, seqs, B, eng.cache, eng.rt, graph_capture=capture,
                          span=self.span)
        h = eng.model.hidden_states(ctx)
        logits = eng.model.logits(h, ctx.want_rows)
        out = torch.empty(B, dtype=torch.int32, device=eng.device)
        native.sample_rows(logits, self.temperature, self.top_k, self.top_p, eng.rng_state, out,
                           ctx.seq_slot)
        return logits, out

    def can_feed_back(self, slots: Sequence[int]) -> bool:
        """Whether the next step of ``slots`` can take the tokens that the latest run sampled
        straight from the device: the graph is recorded and that run was for these slots."""
        return (self.graph is not None and self.out_is_latest
                and self.last_slots == [int(s) for s in slots])

    def run(self, slots: Sequence[int], tokens: Optional[Sequence[int]], use_graph: bool = True):
        """``tokens`` None: the tokens that the latest run sampled, which are still on the
        device (see ``can_feed_back``): the host need not have read them yet."""
        eng, B = self.engine, self.B
        if len(slots) != B or (tokens is not None and len(tokens) != B):
            raise ValueError(f"this graph steps {B} sequences")
        if tokens is None and not (use_graph and self.can_feed_back(slots)):
            raise ValueError("a step can only take its tokens from the device after a replayed "
                             "step of the same sequences")
        V = eng.vocab_size
        for t in tokens or ():
            if not 0 <= int(t) < V:
                raise ValueError(f"input token ID {t} exceeds vocab_size {V}")
        slots = [int(s) for s in slots]
        eng.cache.reserve([(s, 1) for s in slots])
        try:
            result = self._run(slots, tokens, use_graph)
        except BaseException:
            for s in slots:
                eng.cache.trim(s)
            raise
        for s in slots:
            eng.cache.advance(s, 1)
        self.last_slots = slots
        return result

    def _run(self, slots, tokens, use_graph: bool):
        eng, B = self.engine, self.B
        seqs = [(s, eng.cache.length(s), 1) for s in slots]
        stage = self.calls % _STAGES
        if self.copied[stage] is not None:
            self.copied[stage].synchronize()     # (long done unless the caller runs far ahead)
        StepContext.pack_single_tokens(self.host_rows[stage], slots, [st for _, st, _ in seqs],
                                       0 if tokens is None else tokens)
        self.meta.copy_(self.hosts[stage], non_blocking=True)
        if tokens is None:
            self.meta[:B].copy_(self.out, non_blocking=True)     # what the latest replay sampled
        if self.copied[stage] is None:
            self.copied[stage] = torch.cuda.Event()
        self.copied[stage].record()
        eng.cache.sync_tables()
        if self.graph is not None and use_graph:
            self.graph.replay()
            result, self.last_logits = self.out, self.logits
            self.out_is_latest = True
        else:
            self.out_is_latest = False      # (unless this run is recorded below)
            before = native.launch_count()
            # (a step that will be captured runs eagerly under the same rules first, so
            # that a part that cannot be captured fails here, before any recording)
            self.last_logits, result = self._forward(seqs, capture=use_graph)
            self.launches_per_step = native.launch_count() - before
            if use_graph and self.calls >= 1 and native.recording_allowed():
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
                        self.logits, self.out = self._forward(seqs, capture=True)
                finally:
                    if collecting:
                        gc.enable()
                self.graph = g
                # (the recording ran nothing: the tokens of this step, which the next step
                # may be fed with on the device, are put where a replay would have put them)
                self.out.copy_(result)
                self.out_is_latest = True
        self.calls += 1
        return result


class PromptGraph:
    """The step of ``n_seqs`` prompts from position 0 with ``rows`` rows in all (filled up
    with the rows of one more sequence without a slot) and ``n_want`` wanted rows; or, with
    ``from_start=False``, the step of one token for each of ``n_seqs == rows`` sequences
    wherever they stand (nothing to fill up), which returns logits where ``DecodeGraph``
    samples."""

    def __init__(self, engine, rows: int, n_seqs: int, n_want: int, from_start: bool = True,
                 longest: Optional[int] = None, span: Optional[int] = None):
        self.engine = engine
        self.rows, self.B, self.n_want = rows, n_seqs, n_want
        self.span = span
        self.from_start = from_start
        self.longest = longest      # no prompt of a replay is longer (None: no bound but the rows)
        size = StepContext.packed_size(rows, n_seqs + (1 if from_start else 0), n_want)
        self.hosts = [torch.zeros(size, dtype=torch.int32).pin_memory() for _ in range(_STAGES)]
        self.copied = [None] * _STAGES
        self.meta = torch.zeros(size, dtype=torch.int32, device=engine.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.calls = 0
        self.unrecordable: Optional[str] = None     # why recording failed, if it did

    def _forward(self, seqs):
        eng = self.engine
        ctx = StepContext(self.meta, seqs, self.n_want, eng.cache, eng.rt, graph_capture=True,
                          from_start=self.from_start, longest=self.longest, span=self.span)
        return eng.model.logits(eng.model.hidden_states(ctx), ctx.want_rows)

    def run(self, seqs, tokens: np.ndarray, want_rows: Sequence[int]) -> torch.Tensor:
        """``seqs``: ``(slot, start, count)`` of the step's sequences, whose pages are reserved;
        returns the 32-bit logits of the wanted rows, in a buffer that a later run may
        overwrite."""
        eng = self.engine
        used = int(tokens.size)
        if len(seqs) != self.B or len(want_rows) != self.n_want or used > self.rows:
            raise ValueError(f"this graph steps {self.B} sequences of {self.rows} rows in all")
        if self.from_start:
            if self.longest is not None and any(n > self.longest for _, _, n in seqs):
                raise ValueError(f"this graph steps prompts of at most {self.longest} tokens")
            # (the rows that are left over, as sequences without a slot, none longer than the bound)
            padded = list(seqs) + [(-1, 0, self.rows - used)]
            tokens = np.concatenate([tokens, np.zeros(self.rows - used, dtype=np.int64)])
        else:
            if used != self.rows or any(n != 1 for _, _, n in seqs):
                raise ValueError("this graph steps one token for each sequence")
            padded = list(seqs)
        stage = self.calls % _STAGES
        if self.copied[stage] is not None:
            self.copied[stage].synchronize()
        h = self.hosts[stage]
        h.copy_(torch.from_numpy(StepContext.pack(padded, tokens, want_rows)))
        self.meta.copy_(h, non_blocking=True)
        if self.copied[stage] is None:
            self.copied[stage] = torch.cuda.Event()
        self.copied[stage].record()
        eng.cache.sync_tables()
        if self.graph is not None:
            self.graph.replay()
            result = self.logits
        else:
            # Launched one by one, under the rules of a recorded step, the first two times
            # (which warms up what the step uses); the second time the same launches are
            # also recorded for the steps to come, which runs nothing.
            result = self._forward(padded)
            if self.calls >= 1 and native.recording_allowed() and not self.unrecordable:
                g = torch.cuda.CUDAGraph()
                collecting = gc.isenabled()
                gc.collect()
                gc.disable()       # (see DecodeGraph: nothing else may touch CUDA meanwhile)
                try:
                    with torch.cuda.graph(g, capture_error_mode="thread_local"):
                        self.logits = self._forward(padded)
                    self.graph = g
                except RuntimeError as e:
                    # (the step itself has run; steps of this shape stay launched one by one)
                    self.unrecordable = f"{type(e).__name__}: {e}"
                    self.logits = None
                finally:
                    if collecting:
                        gc.enable()
        self.calls += 1
        return result
