"""The engine: model + cache + ONE step function.

``step(entries, want)`` runs exactly the tokens it is given, for sequences
that hold cache slots, as one packed batch (rows of different sequences follow
one another; a recorded short step is filled up with rows of a sequence that
holds no slot, which no other row sees and which are not stored), and
returns 32-bit logits at the wanted rows.  A sequence's first step carries
its whole prompt; later steps carry its next token(s).  Everything above
(generation, replay, benchmarks) goes through this function or through its
graph-captured form for single-token steps, which launches the same kernels.

The reference's step is ``model_forward_step`` for one sequence with one
position counter (src/model/layer.rs:1255-1392); the logits come from a
separate product for one row (src/engine/generate.rs:1097-1126).
"""

from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.paged import SequenceCache
from ..config.registry import read_config_json, spec_from_config
from ..config.spec import ModelSpec
from ..kernels import native
from ..parts.base import Runtime, StepContext
from ..weights.arena import DictSource, FileSource, RandomSource
from .model import DecoderModel, expected_tensors, place_weights

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


class StepError(ValueError):
    pass


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    if dtype not in _DTYPES:
        raise ValueError(f"dtype {dtype!r} is not one of {', '.join(sorted(_DTYPES))}")
    return _DTYPES[dtype]


class Engine:
    """``weights``: a source of the model's stored tensors (``FileSource``,
    ``RandomSource``, ``DictSource``) or a plain ``{name: tensor}`` mapping of them."""

    def __init__(self, spec: ModelSpec, weights, dtype="bfloat16",
                 max_tokens: int = 8192, max_seq_len: Optional[int] = None,
                 page_tokens: int = 64, max_slots: Optional[int] = None, device="cuda:0",
                 max_continuation: Optional[int] = None, where: str = "weights"):
        self.spec = spec
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        native.require_device(self.device)
        torch.cuda.set_device(self.device)
        self.rt = Runtime(self.device, self.dtype)
        spec.validate()
        source = weights if hasattr(weights, "write") else DictSource(weights)
        self.model = DecoderModel(spec, place_weights(spec, source, self.dtype, self.device, where),
                                  self.rt)
        self.max_seq_len = min(max_seq_len or spec.max_positions, spec.max_positions)
        self.cache = SequenceCache(self.model.cache_needs(), max_tokens, self.max_seq_len,
                                   self.dtype, self.device, page_tokens, max_slots,
                                   max_continuation)
        self.vocab_size = spec.vocab_size
        # one xorshift64 state per slot, for the sampling kernel
        self.rng_state = torch.ones(self.cache.max_slots, dtype=torch.int64, device=self.device)
        self.kernel_watch = native.KernelWatch()
        self._graphs: Dict[Tuple, "DecodeGraph"] = {}
        self._prompt_graphs: Dict[Tuple, "PromptGraph"] = {}
        # recorded steps kept, least recently used first out: single-token steps with sampling
        # (by number of sequences, sampling options and length class: recording one costs what
        # 15 replays cost, and each keeps a [sequences, vocabulary] logits buffer), and steps
        # that return logits (prompts by rows, sequences and wanted rows; tokens likewise)
        self.max_graphs = 48
        self.max_prompt_graphs = 16
        self.first_span = 512       # the shortest length class of recorded single-token steps
        self.prompt_graph_rows = 1024   # steps of prompts of up to this many rows are recorded
        self.last_logits: Optional[torch.Tensor] = None   # of the latest sampled step
        self._latest_step = None    # key of the recorded single-token step that ran last, if one did
        self._read_ring = None      # pinned buffers and events of read_later, made at first use
        self._reads = 0

    # ---- construction ----------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str, dtype="bfloat16", **kw) -> "Engine":
        """Load ``config.json`` and the safetensors of ``model_dir``; the model is
        chosen by the architecture named in config.json."""
        from ..weights.safetensors_io import ModelFiles
        config = read_config_json(model_dir)
        _, spec = spec_from_config(config)
        native.require_device(torch.device(kw.get("device", "cuda:0")))
        return cls(spec, FileSource(ModelFiles(model_dir)), dtype, where=model_dir, **kw)

    @classmethod
    def from_random(cls, config: Mapping, seed: int, dtype="bfloat16", matrix_std: float = None,
                    norm_std: float = None, store=None, **kw) -> "Engine":
        """Seeded random weights drawn on the device straight into the weight buffer (no
        files, no host copy): the model ``write_random_model(dir, config, seed, store)``
        writes, tensor for tensor and bit for bit.  ``store`` is the type the folder would
        hold (default: the compute type); bfloat16 weights run in 32-bit are the check path
        of a bfloat16 model."""
        from ..weights import random_init
        _, spec = spec_from_config(config)
        native.require_device(torch.device(kw.get("device", "cuda:0")))
        source = RandomSource(expected_tensors(spec), seed, parse_dtype(store or dtype),
                              random_init.MATRIX_STD if matrix_std is None else matrix_std,
                              random_init.NORM_STD if norm_std is None else norm_std)
        return cls(spec, source, dtype, **kw)

    # ---- sequences -------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.acquire()

    def end_sequence(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step --------------------------------------------------------
    def _prepare(self, entries: Sequence[Tuple[int, Sequence[int]]],
                 want: Optional[Sequence[Sequence[int]]]):
        """The step's sequences ``[(slot, start, count)]``, its token ids (one array) and
        the packed indices of its wanted rows, all checked; nothing is reserved yet."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        slots = [int(s) for s, _ in entries]
        if len(set(slots)) != len(slots):
            raise StepError("a sequence appears twice in one step")
        counts = [len(t) for _, t in entries]
        if min(counts) <= 0:
            raise StepError("every sequence of a step needs at least one token")
        V = self.vocab_size
        tokens = np.concatenate([np.asarray(toks, dtype=np.int64).reshape(-1) for _, toks in entries])
        if tokens.size and not (0 <= tokens.min() and tokens.max() < V):
            bad = tokens[(tokens < 0) | (tokens >= V)][0]
            raise StepError(f"input token ID {bad} exceeds vocab_size {V}")
        starts = [self.cache.length(s) for s in slots]
        if any(st > 0 for st in starts):
            # (a step of prompts only attends over its own rows and may be of any length)
            for slot, st, n in zip(slots, starts, counts):
                most = self.cache.max_step_tokens(st)
                if n > most:
                    raise StepError(
                        f"slot {slot}: a step that continues sequences may add at most {most} "
                        f"positions to a sequence of {st} (the windowed layers keep "
                        f"the window and room for {self.cache.max_step_tokens()} more; "
                        f"'max_continuation' sizes that room); got {n}")
        if want is None:
            want = [[c - 1] for c in counts]
        if len(want) != len(entries):
            raise StepError("'want' needs one list per sequence")
        want_rows, row0 = [], 0
        for b, c in enumerate(counts):
            for w in want[b]:
                if not 0 <= int(w) < c:
                    raise StepError(f"wanted place {w} is outside the {c} tokens "
                                    f"of its sequence")
                want_rows.append(row0 + int(w))
            row0 += c
        return list(zip(slots, starts, counts)), tokens, want_rows

    def _context(self, entries: Sequence[Tuple[int, Sequence[int]]],
                 want: Optional[Sequence[Sequence[int]]]):
        seqs, tokens, want_rows = self._prepare(entries, want)
        self.cache.reserve([(s, n) for s, _, n in seqs])
        return self._step_context(seqs, tokens, want_rows)

    def _step_context(self, seqs, tokens, want_rows) -> StepContext:
        host = torch.from_numpy(StepContext.pack(seqs, tokens, want_rows)).pin_memory()
        meta = host.to(self.device, non_blocking=True)
        return StepContext(meta, seqs, len(want_rows), self.cache, self.rt)

    def _recorded_prompts(self, seqs, n_rows: int, n_want: int) -> bool:
        """Whether this step goes through a recorded prompt step: prompts from position 0
        with more rows than the few-row kernels take and so few that launching them one by
        one costs more than running them, and few wanted rows (a recorded step keeps a
        logits buffer of that many rows)."""
        return (self.prompt_graph_rows > 0 and self.model.captures_prompts
                and self.rt.fused_rope_max_rows < n_rows <= self.prompt_graph_rows
                and 0 < n_want <= 64 and all(st == 0 for _, st, _ in seqs))

    def _recorded_tokens(self, seqs, n_want: int) -> bool:
        """Whether this step goes through a recorded single-token step that returns logits:
        one token for every sequence, few wanted rows, parts that may be recorded."""
        return (self.prompt_graph_rows > 0 and self.model.captures_prompts
                and len(seqs) <= self.prompt_graph_rows and 0 < n_want <= 64
                and all(n == 1 for _, _, n in seqs))

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Run one step.

        ``entries``: ``(slot, tokens)`` per sequence; the tokens continue the
        sequence from its current length.  ``want``: per sequence, the places
        among ITS tokens of this step whose logits are returned (default: the
        last).  Returns ``[n_wanted, vocab]`` 32-bit logits on the device, in the
        order of the entries and of ``want`` (``None`` if nothing is wanted).

        Short steps of prompts are recorded into a CUDA graph the second time their shape
        (rows rounded up to 64, sequences, wanted rows) is seen and replayed from then on
        (``prompt_graph_rows``: the most rows of such a step; 0: none are recorded); so are
        steps of one token for every sequence, by the number of sequences and wanted rows.
        """
        seqs, tokens, want_rows = self._prepare(entries, want)
        self._latest_step = None        # (no later step may be fed with an earlier step's tokens)
        self.cache.reserve([(s, n) for s, _, n in seqs])
        try:
            if self._recorded_prompts(seqs, int(tokens.size), len(want_rows)):
                logits = self._prompt_step(seqs, tokens, want_rows)
            elif self._recorded_tokens(seqs, len(want_rows)):
                logits = self._prompt_step(seqs, tokens, want_rows, from_start=False)
            else:
                ctx = self._step_context(seqs, tokens, want_rows)
                self.cache.sync_tables()
                h = self.model.hidden_states(ctx)
                logits = self.model.logits(h, ctx.want_rows) if ctx.want_rows.numel() else None
        except BaseException:
            for slot, _, _ in seqs:      # hand back the pages reserved for the failed step
                self.cache.trim(slot)
            raise
        for slot, _, n in seqs:
            self.cache.advance(slot, n)
        return logits

    def _prompt_step(self, seqs, tokens, want_rows, from_start: bool = True) -> torch.Tensor:
        from .graph import PromptGraph
        rows = -(-int(tokens.size) // 64) * 64 if from_start else int(tokens.size)
        # (steps whose prompts are all short are recorded apart: their attention is another kernel)
        short = self.rt.short_prompt_tokens
        longest = short if from_start and max(n for _, _, n in seqs) <= short < rows else None
        span = None if from_start else self._span([s for s, _, _ in seqs])
        key = ("prompts" if from_start else "tokens", rows, len(seqs), len(want_rows), longest, span)
        g = self._prompt_graphs.pop(key, None)
        if g is None:
            g = PromptGraph(self, rows, len(seqs), len(want_rows), from_start, longest, span)
            while len(self._prompt_graphs) >= self.max_prompt_graphs:
                self._prompt_graphs.pop(next(iter(self._prompt_graphs)))
        self._prompt_graphs[key] = g       # most recently used last
        # (the graph's buffer is overwritten by its next replay: the caller gets a copy)
        return g.run(seqs, tokens, want_rows).clone()

    # ---- sampling --------------------------------------------------------
    def seed_sequence(self, slot: int, seed: int) -> None:
        """Set the slot's generator (0 becomes 1, src/engine/sampler.rs:38-42)."""
        seed = int(seed) & 0xFFFFFFFFFFFFFFFF
        if seed == 0:
            seed = 1
        if seed >= 1 << 63:
            seed -= 1 << 64
        self.rng_state[slot] = seed

    def sample(self, logits: torch.Tensor, slots: Sequence[int], temperature: float = 0.0,
               top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
        """One token per row of ``logits``; row i draws from the generator of ``slots[i]``."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        index = torch.tensor(list(slots), dtype=torch.int32).to(logits.device)
        return native.sample_rows(logits, temperature, top_k, top_p, self.rng_state, out, index)

    # ---- single-token steps through a captured graph ----------------------
    def decode_step(self, slots: Sequence[int], tokens: Optional[Sequence[int]],
                    temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                    use_graph: bool = True) -> torch.Tensor:
        """One token for each of ``slots``, then one sampled token each: the
        same kernels as ``step`` + ``sample``, replayed from a CUDA graph that
        is captured the second time a batch size is seen.  Returns the sampled
        tokens as an int32 tensor on the device (the next step of the same graph
        overwrites it).  ``tokens`` None: the tokens that the step before sampled for the
        same slots, taken on the device (``can_feed_back`` says whether that is possible);
        the host may read them afterwards."""
        from .graph import DecodeGraph
        key = (len(slots), float(temperature), int(top_k), float(top_p), self._span(slots))
        g = self._graphs.pop(key, None)
        if g is None:
            g = DecodeGraph(self, *key)
            while len(self._graphs) >= self.max_graphs:
                # the least recently used one goes, with its buffers (each holds a
                # [sequences, vocab] 32-bit logits buffer beside its activations)
                self._graphs.pop(next(iter(self._graphs)))
        self._graphs[key] = g       # most recently used last
        if tokens is None and self._latest_step != key:
            raise StepError("a step can take its tokens from the device only right after a step "
                            "of the same sequences through the same recorded step")
        self._latest_step = None
        out = g.run(slots, tokens, use_graph)
        self._latest_step = key
        self.last_logits = g.last_logits
        return out

    def can_feed_back(self, slots: Sequence[int], temperature: float = 0.0, top_k: int = 0,
                      top_p: float = 1.0) -> bool:
        """Whether ``decode_step(slots, None, ...)`` is possible now."""
        key = (len(slots), float(temperature), int(top_k), float(top_p), self._span(slots))
        g = self._graphs.get(key)
        return g is not None and self._latest_step == key and g.can_feed_back(slots)

    def recorded_step(self, n_seqs: int, temperature: float = 0.0, top_k: int = 0,
                      top_p: float = 1.0):
        """The most recently used recorded single-token step for this many sequences and these
        sampling options (of whatever length class), or None."""
        want = (n_seqs, float(temperature), int(top_k), float(top_p))
        for key in reversed(list(self._graphs)):
            if key[:4] == want:
                return self._graphs[key]
        return None

    def _span(self, slots: Sequence[int]) -> int:
        """The length class of a single-token step: the next power of two (from 512 on) that
        holds the longest of its sequences after the step.  A recorded step divides the
        attention's work for that length; sequences that outgrow it move on to the next
        class's recording."""
        longest = max(self.cache.length(int(s)) for s in slots) + 1
        span = self.first_span
        while span < longest:
            span *= 2
        return min(span, self.max_seq_len)

    def read_later(self, t: torch.Tensor):
        """Start bringing the integer tensor ``t`` (at most one value per slot) to the host:
        the copy is enqueued now, behind the step that makes ``t`` and ahead of whatever is
        launched next; ``read_now`` of the returned ticket waits for it."""
        n = t.numel()
        if self._read_ring is None:
            self._read_ring = [(torch.zeros(self.cache.max_slots, dtype=torch.int32).pin_memory(),
                                torch.cuda.Event()) for _ in range(4)]
        buf, event = self._read_ring[self._reads % len(self._read_ring)]
        self._reads += 1
        buf[:n].copy_(t.reshape(-1), non_blocking=True)
        self.kernel_watch.fetch()
        event.record()
        return buf, n, event

    def read_now(self, ticket) -> List[int]:
        """The values of a ``read_later`` ticket, and the check that no kernel so far gave up
        on a bounded wait.  At most four tickets may be open at a time."""
        buf, n, event = ticket
        event.synchronize()
        self.kernel_watch.check()
        return buf[:n].tolist()

    def read_back(self, t: torch.Tensor):
        """``t`` on the host (a list for integer tensors, else a tensor), and a check that
        no kernel of the steps so far gave up on a bounded wait: the error words ride on
        the same stream and the same synchronisation as the copy of ``t``."""
        self.kernel_watch.fetch()
        out = t.tolist() if not t.dtype.is_floating_point else t.cpu()
        self.kernel_watch.check()
        return out

    def memory_report(self) -> dict:
        return {"weights_bytes": self.model.weight_bytes(), "cache_bytes": self.cache.bytes(),
                "cache_tokens": self.cache.max_tokens, "slots": self.cache.max_slots}
