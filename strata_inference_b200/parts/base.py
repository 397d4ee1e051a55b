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
``Embedding``
    ``tensors(params, hidden, vocab)``, ``forward(ctx) -> h``: the step's rows of the
    32-bit residual stream from ``ctx.tokens`` (and ``ctx.row_pos`` if it adds positions).
``Block``
    ``forward(h, normed, ctx, entry, cache_entry, owns_cache, next_norm)``:
    ``h`` is the 32-bit residual stream, updated in place; ``normed`` is
    ``first_norm(h)`` if the previous block already made it; the block returns
    ``next_norm(h)`` when it can fuse that, else ``None``.

Tensors.  ``tensors(...)`` declares what a model folder stores for the part.  A part may
also declare ``resident(...)`` (same arguments): what it keeps on the device and how that
is put together from the stored tensors (weights/arena.py); its constructor then gets the
resident tensors, already in place in the model's one weight buffer.  Without
``resident`` it gets every stored tensor under its stored name, in its stored type.
``build_part`` builds one part alone from stored tensors.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.paged import KVView, SequenceCache
from ..kernels import native
from ..weights.arena import DictSource, WeightArena, resident_of


class Runtime:
    """Device, compute type and the matrix product, shared by all parts."""

    def __init__(self, device, dtype: torch.dtype):
        self.device = torch.device(device)
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute type must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        native.require_device(self.device)
        native.library()
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # true 32-bit products: no reduced-precision matrix mode anywhere
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")
        # Up to this many rows a product goes to the weight-streaming kernel (which takes up
        # to native.SKINNY_MAX_ROWS).  Measured inside decode steps on a B200: with 9 to 16
        # rows (two activation tiles per warp) the library product is ahead, by 3-9 % of the
        # step at Gemma2-2B sizes, 9 % at 9B and 16 % at 27B sizes (batch 16); with up to 8
        # rows the kernel is far ahead (a layer's products: 45 us against 66 us).
        self.skinny_max_rows = 8
        # The q|k|v product that rotates and stores in its epilogue stays ahead of the
        # library product followed by the rotation kernel up to 16 rows (and behind from 17).
        self.fused_rope_max_rows = 16
        self.chain_max_rows = 16     # what the (optional) chain kernel of few-row steps takes
        # prompts of up to this many tokens are attended to by the mma.sync prompt kernel
        self.short_prompt_tokens = 128
        # a step that continues a sequence with at least this many tokens attends through the
        # prompt kernel over a packed copy of what the sequence holds (parts/attention.py)
        self.piece_attention_rows = 32
        # Up to 128 rows against a matrix of so many rows that its 128-row tiles are several
        # waves of blocks go to the tcgen05 weight-streaming product (csrc/linear_rows_tc.cu):
        # there it reads at 0.91 of the copy bandwidth; with fewer tiles the library is as fast.
        self.rows_tc_max_rows = native.linear_rows_tc_max_rows()
        self.rows_tc_min_weight_rows = 4 * 128 * self.sm_count
        # SIB_LINEAR_STREAM=1: few-row products go to the kernel that stages its weights through
        # shared memory (csrc/linear_stream.cu) instead of the one that loads them straight
        # into registers.  Alone it is the faster of the two on most shapes; inside a chained
        # step it is slower (2B shape, batch 8: 3.29 against 2.51 ms), because a block of it
        # needs a third of an SM's shared memory before it can start under its predecessor.
        self.stream_products = os.environ.get("SIB_LINEAR_STREAM", "0")
        # SIB_FUSE_ROTATION=0: rotation and cache write always run as a kernel of their own
        self.fuse_rotation = os.environ.get("SIB_FUSE_ROTATION", "1") != "0"
        # from this many rows on the gate/up product with its gated epilogue (pairs of SMs,
        # 256 x 256 tiles) beats the library product followed by the activation kernel
        self.gated_gemm_min_rows = 128
        # SIB_EARLY_KEYS=0: the attention over the cache fetches no keys before the kernel ahead
        # of it has finished
        self.early_keys = os.environ.get("SIB_EARLY_KEYS", "1") != "0"
        # SIB_DECODE_CHAIN=1: the steps between two attention kernels of a step of few rows run
        # as ONE chain kernel (csrc/decode_chain.cu) instead of one kernel each.  Measured on
        # the Gemma2-2B shape it is the slower of the two so far (a layer's products and norms:
        # 60 against 47 us at batch 8), so it is off unless asked for.
        self.chain_steps = os.environ.get("SIB_DECODE_CHAIN", "0") == "1"
        self.chain: Optional[ProductChain] = None
        self._chain_sync: Optional[torch.Tensor] = None
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

    # ---- chains of deferred steps ------------------------------------------
    def chaining(self, rows: int):
        """A context in which the few-row products and the "norm, add, norm" steps issued
        through this runtime are collected and run as ONE kernel (csrc/decode_chain.cu) as
        soon as anything else is launched through ``kernels.native`` (or the context ends).
        Results of deferred steps are tensors like any other, but their contents exist only
        after the chain ran: code that reads them with anything but this runtime's methods
        or the launchers of ``kernels.native`` calls ``flush()`` first.  Blocks whose parts
        do not promise that (``chain_safe``) run with the chain suspended."""
        return _Chaining(self, rows)

    def flush(self) -> None:
        if self.chain is not None:
            self.chain.flush()

    def chain_sync(self) -> torch.Tensor:
        if self._chain_sync is None:
            self._chain_sync = torch.zeros(2, dtype=torch.int32, device=self.device)
        return self._chain_sync

    def _chainable(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> bool:
        R, K = x.shape
        return (self.chain is not None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and 0 < R <= self.chain.rows and K % 8 == 0 and x.stride(1) == 1
                and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()
                and out_dtype in (torch.bfloat16, torch.float32))

    def linear_rope(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, **rope) -> torch.Tensor:
        """The q|k|v product of few rows that rotates q and k and writes k and v into the
        cache (``native.skinny_linear_rope``'s arguments by name), deferred when a chain is
        being collected."""
        if self._chainable(x, w, out.dtype):
            self.chain.add(native.chain_product(x, w, out, rope=rope), (x, w, out))
            return out
        return native.skinny_linear_rope(
            x, w, out, rope["row_pos"], rope["row_seq"], rope["seq_slot"], rope["seq_end"],
            rope["inv_freq"], rope["k_pool"], rope["v_pool"], rope["page_table"],
            rope["page_tokens"], rope["ring_tokens"], rope["n_heads"], rope["n_kv"],
            rope["head_dim"])

    def add_rms_norm(self, a: torch.Tensor, post_gain, post_eps: float, h: torch.Tensor, pre_gain,
                     pre_eps: float, out: Optional[torch.Tensor]) -> None:
        """``native.add_rms_norm``, deferred when a chain is being collected."""
        if (self.chain is not None and a.dtype == torch.bfloat16 and a.stride(1) == 1
                and a.shape[0] <= self.chain.rows and (out is None or out.stride(1) == 1)):
            self.chain.add(native.chain_norm(a, post_gain, post_eps, h, pre_gain, pre_eps, out),
                           (a, h, out))
            return
        native.add_rms_norm(a, post_gain, post_eps, h, pre_gain, pre_eps, out)

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
        if self._chainable(x, w, out_dtype) and (out_dtype == torch.bfloat16
                                                 or epilogue != native.EPI_GEGLU):
            out = torch.empty((R, n_out), dtype=out_dtype, device=x.device)
            self.chain.add(native.chain_product(x, w, out, epilogue, cap), (x, w, out))
            return out
        self.flush()        # (a library product below is not launched through kernels.native)
        if (x.dtype == torch.bfloat16 and 0 < R <= self.skinny_max_rows and K % 8 == 0
                and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0):
            out = torch.empty((R, n_out), dtype=out_dtype, device=x.device)
            mode = self.stream_products
            if mode == "1" or (mode == "down" and K >= 2 * N) or (mode == "small" and N * K < 30e6) \
                    or (mode == "notgu" and epilogue != native.EPI_GEGLU and N < 100000):
                return native.linear_stream(x, w, out, epilogue, cap)
            return native.skinny_linear(x, w, out, epilogue, cap)
        aligned = (K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                   and x.data_ptr() % 16 == 0)
        if (x.dtype == torch.bfloat16 and aligned and R <= self.rows_tc_max_rows
                and N >= self.rows_tc_min_weight_rows and w.is_contiguous()):
            # some rows against very many weight rows (the logits of a batch of 17 to 128):
            # the weight-streaming tcgen05 product, with its epilogue
            out = torch.empty((R, n_out), dtype=out_dtype, device=x.device)
            return native.linear_rows_tc(x, w, out, epilogue, cap)
        fused_gate = epilogue == native.EPI_GEGLU and R > self.gated_gemm_min_rows
        if x.dtype == torch.bfloat16 and aligned and (out_dtype == torch.float32 or fused_gate):
            # the tcgen05 product where its epilogue saves a pass over the outputs: 32-bit
            # logits of many rows, soft-capped as they are written; the gated activation of
            # the feed-forward, which halves what is written and spares a second kernel
            out = torch.empty((R, n_out), dtype=out_dtype, device=x.device)
            return native.gemm_tcgen05(x, w, out, epilogue, cap)
        if epilogue == native.EPI_GEGLU:
            raise ValueError("the gated epilogue exists in the hand-written products only")
        with native.profile_region(f"library product {N}x{K}",
                                   (N * K + R * K) * x.element_size() + R * N * 4,
                                   2.0 * R * N * K):
            if out_dtype == x.dtype:
                y = torch.matmul(x, w.t())
            else:
                y = torch.mm(x, w.t(), out_dtype=out_dtype)
        if epilogue == native.EPI_SOFTCAP:
            if y.dtype != torch.float32:
                raise ValueError("the soft cap epilogue is applied to 32-bit outputs")
            native.softcap_(y, cap)
        return y


class ProductChain:
    """Deferred few-row steps, in the order they were issued, run as one kernel."""

    def __init__(self, rt: Runtime, rows: int):
        self.rt = rt
        self.rows = rows
        self.phases: list = []
        self.keep: list = []          # the steps' tensors, alive until the kernel is launched
        self.most = native.decode_chain_max_phases()

    def add(self, phase, tensors) -> None:
        if len(self.phases) == self.most:
            self.flush()
        self.phases.append(phase)
        self.keep.append(tensors)

    def flush(self) -> None:
        if not self.phases:
            return
        # (the steps' tensors stay referenced until the kernel is launched: memory that is
        # handed back earlier could be given to someone else, and written, before it runs)
        phases, keep = self.phases, self.keep
        self.phases, self.keep = [], []
        native.decode_chain(phases, self.rows, self.rt.chain_sync())
        del keep


class _Chaining:
    def __init__(self, rt: Runtime, rows: int):
        self.rt, self.rows = rt, rows

    def __enter__(self) -> ProductChain:
        self.outer = self.rt.chain
        if self.outer is not None:
            self.outer.flush()
        self.rt.chain = ProductChain(self.rt, self.rows)
        native.set_pending(self.rt.chain.flush)
        return self.rt.chain

    def __exit__(self, exc_type, exc, tb) -> None:
        chain, self.rt.chain = self.rt.chain, self.outer
        native.set_pending(self.outer.flush if self.outer is not None else None)
        if exc_type is None:
            chain.flush()


class _ChainSuspended:
    """Runs a part that does not know about deferred steps: what was collected goes
    first, and nothing is deferred meanwhile."""

    def __init__(self, rt: Runtime):
        self.rt = rt

    def __enter__(self) -> None:
        self.chain = self.rt.chain
        if self.chain is not None:
            self.chain.flush()
            self.rt.chain = None
            native.set_pending(None)

    def __exit__(self, *exc) -> None:
        if self.chain is not None:
            self.rt.chain = self.chain
            native.set_pending(self.chain.flush)


def chain_suspended(rt: Runtime) -> _ChainSuspended:
    return _ChainSuspended(rt)


class CapturedStepError(RuntimeError):
    """A part read a host-side value of a step that is being captured into a CUDA graph."""


_ORDER: Dict[int, np.ndarray] = {}      # 0..B-1 by B


class StepContext:
    """One step's rows: which sequence and position each row is, on the device for the
    kernels and on the host for launch decisions.

    There is one way to make one: ``pack`` lays a step's integers out as
    ``[tokens R | row_pos R | row_seq R | seq_slot B | seq_start B | seq_end B |
    seq_row0 B | wanted rows n]`` (R rows, B sequences), the caller brings that array to
    the device, and the constructor cuts the views.  The engine's step, the captured
    single-token step and the tests all go through it.

    A *captured* step (``graph_capture=True``) is recorded once and replayed for other
    sequences, positions and slots: only the device tensors are refreshed before a replay.
    What is the same in every replay stays readable on the host (``n_rows``, ``n_seqs``,
    ``max_count``, ``all_from_start``, and ``counts`` of single-token steps); reading
    ``starts``, ``slots`` or ``max_end`` raises :class:`CapturedStepError`, because a value
    read while recording would be frozen into the graph.  A part that is to run in captured
    steps indexes its cache or state with the device tensors (``seq_slot``, ``row_pos``,
    ...) only.

    A captured step of prompts (``from_start=True``) is replayed for other prompts with the
    same number of sequences and at most as many rows in all: its last sequence holds no
    slot (``seq_slot`` -1) and takes the rows that are left over, nothing of it is stored,
    and ``counts`` is not readable either; ``max_count`` is the number of rows, the most
    that one sequence of a replay can have, or the smaller bound ``longest`` that the caller
    keeps for every replay.
    """

    @staticmethod
    def pack(seqs: Sequence[Tuple[int, int, int]], tokens, want_rows: Sequence[int] = ()) -> np.ndarray:
        """The step's integers (an int32 array) for sequences ``[(slot, start, count)]``;
        ``tokens`` are the R token ids in packed order (None: zeros)."""
        B = len(seqs)
        sq = np.asarray(seqs, dtype=np.int64).reshape(B, 3)
        slots, starts, counts = sq[:, 0], sq[:, 1], sq[:, 2]
        row0 = np.cumsum(counts) - counts
        R = int(counts.sum())
        row_seq = np.repeat(np.arange(B, dtype=np.int64), counts)
        row_pos = np.arange(R, dtype=np.int64) - row0[row_seq] + starts[row_seq]
        toks = np.zeros(R, dtype=np.int64) if tokens is None else np.asarray(tokens, dtype=np.int64)
        if toks.shape != (R,):
            raise ValueError(f"{toks.size} tokens for {R} rows")
        want = np.asarray(list(want_rows), dtype=np.int64)
        return np.concatenate([toks, row_pos, row_seq, slots, starts, starts + counts, row0,
                               want]).astype(np.int32)

    @staticmethod
    def pack_single_tokens(out: np.ndarray, slots: Sequence[int], lengths: Sequence[int],
                           tokens: Sequence[int]) -> None:
        """What ``pack`` gives for a step of one token for each of B sequences with every
        row wanted, written into ``out`` (int32, [8, B]: the eight runs of the layout, each
        of length B here) without making arrays on the way: the step that is taken
        thousands of times in a row."""
        order = _ORDER.get(len(slots))
        if order is None:
            order = _ORDER[len(slots)] = np.arange(len(slots), dtype=np.int32)
        out[0] = tokens
        out[1] = out[4] = lengths
        out[2] = out[6] = out[7] = order
        out[3] = slots
        out[5] = out[4] + 1

    @staticmethod
    def packed_size(n_rows: int, n_seqs: int, n_want: int) -> int:
        return 3 * n_rows + 4 * n_seqs + n_want

    def __init__(self, meta: torch.Tensor, seqs: Sequence[Tuple[int, int, int]], n_want: int,
                 cache: SequenceCache, runtime: Runtime, graph_capture: bool = False,
                 from_start: bool = False, longest: Optional[int] = None,
                 span: Optional[int] = None):
        """``graph_capture`` with ``from_start``: a captured step of prompts that all start at
        position 0 (replays bring other prompts of at most this step's rows in all, filled up
        with the rows of a sequence that holds no slot: slot -1, nothing of it is stored)."""
        self.n_seqs = B = len(seqs)
        self._counts = [int(n) for _, _, n in seqs]
        self.n_rows = R = sum(self._counts)
        if meta.numel() < self.packed_size(R, B, n_want):
            raise ValueError("the packed step is shorter than its rows and sequences need")
        at = [0]

        def take(n: int) -> torch.Tensor:
            v = meta[at[0]:at[0] + n]
            at[0] += n
            return v
        self.tokens = take(R)        # [rows] int32
        self.row_pos = take(R)       # [rows] absolute position of the row
        self.row_seq = take(R)       # [rows] index of the row's sequence in this step
        self.seq_slot = take(B)      # [seqs] cache slot
        self.seq_start = take(B)     # [seqs] length before the step
        self.seq_end = take(B)       # [seqs] length after the step
        self.seq_row0 = take(B)      # [seqs] packed index of the sequence's first row
        self.want_rows = take(n_want)
        # (the most rows of one sequence sizes launches: a captured step of prompts may be
        # replayed with one sequence that takes nearly all rows)
        # ``span``: how long the sequences of a recorded step's replays get at most, if the
        # caller says (work is divided for that length; any length stays correct)
        self.span = span if graph_capture else None
        # (``longest``: a bound that the caller promises for every replay)
        self.max_count = (longest or R) if (graph_capture and from_start) else max(self._counts)
        self.graph_capture = graph_capture
        self._counts_vary = graph_capture and from_start
        self.all_from_start = from_start if graph_capture else all(st == 0 for _, st, _ in seqs)
        self._starts = [int(st) for _, st, _ in seqs]
        self._slots = [int(s) for s, _, _ in seqs]
        self._max_end = max(st + n for _, st, n in seqs)
        self.cache = cache
        self.runtime = runtime
        self.memo: Dict = {}       # what parts work out once a step (kept by their own keys)

    def _host(self, name: str, value):
        if self.graph_capture:
            raise CapturedStepError(
                f"'{name}' was read on the host while the step is captured into a CUDA graph; "
                f"a replay runs other sequences, so captured steps may use the device "
                f"tensors of the context only")
        return value

    @property
    def counts(self) -> List[int]:
        """Rows per sequence (in a captured step of prompts they change between replays)."""
        return self._host("counts", self._counts) if self._counts_vary else self._counts

    @property
    def starts(self) -> List[int]:
        return self._host("starts", self._starts)

    @property
    def slots(self) -> List[int]:
        return self._host("slots", self._slots)

    @property
    def max_end(self) -> int:
        return self._host("max_end", self._max_end)

    def kv(self, entry: int) -> KVView:
        return self.cache.kv_view(entry)

    def state(self, entry: int) -> torch.Tensor:
        return self.cache.state_view(entry)


def build_part(part_class, args: Tuple, stored, rt: Runtime, *extra):
    """One part alone, from its stored tensors: ``part_class(*args, tensors, rt, *extra)``
    with the part's resident tensors put together as the model's loader does it."""
    plan = {name: (res, "") for name, res in
            resident_of(part_class, part_class.tensors(*args), *args).items()}
    arena = WeightArena(plan, rt.dtype, rt.device, {n: t.dtype for n, t in stored.items()})
    arena.fill(DictSource(stored))
    return part_class(*args, arena.tensors, rt, *extra)
