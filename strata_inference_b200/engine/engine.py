"""The engine: model + cache + ONE step function.

``step(entries, want)`` runs exactly the tokens it is given, for sequences
that hold cache slots, as one packed batch (no padding rows exist), and
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

import torch

from ..cache.paged import SequenceCache
from ..config.registry import read_config_json, spec_from_config
from ..config.spec import ModelSpec
from ..kernels import native
from ..parts.base import Runtime, StepContext
from ..weights.loader import load_weights
from .model import DecoderModel, expected_tensors

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
    def __init__(self, spec: ModelSpec, weights: Mapping[str, torch.Tensor], dtype="bfloat16",
                 max_tokens: int = 8192, max_seq_len: Optional[int] = None,
                 page_tokens: int = 64, max_slots: Optional[int] = None, device="cuda:0"):
        self.spec = spec
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.rt = Runtime(self.device, self.dtype)
        self.model = DecoderModel(spec, weights, self.rt)
        self.max_seq_len = min(max_seq_len or spec.max_positions, spec.max_positions)
        self.cache = SequenceCache(self.model.cache_needs(), max_tokens, self.max_seq_len,
                                   self.dtype, self.device, page_tokens, max_slots)
        self.vocab_size = spec.vocab_size
        # one xorshift64 state per slot, for the sampling kernel
        self.rng_state = torch.ones(self.cache.max_slots, dtype=torch.int64, device=self.device)
        self._graphs: Dict[Tuple, "DecodeGraph"] = {}
        self.last_logits: Optional[torch.Tensor] = None   # of the latest sampled step

    # ---- construction ----------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str, dtype="bfloat16", **kw) -> "Engine":
        """Load ``config.json`` and the safetensors of ``model_dir``; the model is
        chosen by the architecture named in config.json."""
        config = read_config_json(model_dir)
        _, spec = spec_from_config(config)
        device = torch.device(kw.get("device", "cuda:0"))
        native.require_device(device)
        weights = load_weights(model_dir, expected_tensors(spec), device)
        return cls(spec, weights, dtype, **kw)

    @classmethod
    def from_random(cls, config: Mapping, seed: int, dtype="bfloat16", **kw) -> "Engine":
        """Random weights drawn on the device (no files): for benchmarks of large shapes."""
        from ..weights.random_init import random_tensors
        _, spec = spec_from_config(config)
        device = torch.device(kw.get("device", "cuda:0"))
        native.require_device(device)
        weights = random_tensors(expected_tensors(spec), seed, parse_dtype(dtype), device)
        return cls(spec, weights, dtype, **kw)

    # ---- sequences -------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.acquire()

    def end_sequence(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step --------------------------------------------------------
    def _context(self, entries: Sequence[Tuple[int, Sequence[int]]],
                 want: Optional[Sequence[Sequence[int]]]):
        if not entries:
            raise StepError("a step needs at least one sequence")
        slots = [int(s) for s, _ in entries]
        if len(set(slots)) != len(slots):
            raise StepError("a sequence appears twice in one step")
        counts = [len(t) for _, t in entries]
        if min(counts) <= 0:
            raise StepError("every sequence of a step needs at least one token")
        V = self.vocab_size
        for _, toks in entries:
            for t in toks:
                if not 0 <= int(t) < V:
                    raise StepError(f"input token ID {t} exceeds vocab_size {V}")
        starts = [self.cache.length(s) for s in slots]
        all_from_start = all(st == 0 for st in starts)
        if not all_from_start and max(counts) > self.cache.max_step_tokens():
            raise StepError(f"a step that continues sequences may add at most "
                            f"{self.cache.max_step_tokens()} positions to each; "
                            f"got {max(counts)}")
        if want is None:
            want = [[c - 1] for c in counts]
        if len(want) != len(entries):
            raise StepError("'want' needs one list per sequence")
        self.cache.reserve(list(zip(slots, counts)))

        R, B = sum(counts), len(entries)
        row0, acc = [], 0
        for c in counts:
            row0.append(acc)
            acc += c
        tokens, row_pos, row_seq, want_rows = [], [], [], []
        for b, (_, toks) in enumerate(entries):
            tokens.extend(int(t) for t in toks)
            row_pos.extend(range(starts[b], starts[b] + counts[b]))
            row_seq.extend([b] * counts[b])
            for w in want[b]:
                if not 0 <= int(w) < counts[b]:
                    raise StepError(f"wanted place {w} is outside the {counts[b]} tokens "
                                    f"of its sequence")
                want_rows.append(row0[b] + int(w))
        ends = [s + c for s, c in zip(starts, counts)]
        flat = tokens + row_pos + row_seq + slots + starts + ends + row0 + want_rows
        host = torch.tensor(flat, dtype=torch.int32).pin_memory()
        meta = host.to(self.device, non_blocking=True)
        o = [0]

        def take(n):
            v = meta[o[0]:o[0] + n]
            o[0] += n
            return v
        ctx = StepContext(
            n_rows=R, n_seqs=B, tokens=take(R), row_pos=take(R), row_seq=take(R),
            seq_slot=take(B), seq_start=take(B), seq_end=take(B), seq_row0=take(B),
            starts=starts, counts=counts, slots=slots, all_from_start=all_from_start,
            max_count=max(counts), max_end=max(ends), cache=self.cache, runtime=self.rt)
        return ctx, take(len(want_rows))

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Run one step.

        ``entries``: ``(slot, tokens)`` per sequence; the tokens continue the
        sequence from its current length.  ``want``: per sequence, the places
        among ITS tokens of this step whose logits are returned (default: the
        last).  Returns ``[n_wanted, vocab]`` 32-bit logits on the device, in the
        order of the entries and of ``want`` (``None`` if nothing is wanted).
        """
        ctx, want_rows = self._context(entries, want)
        self.cache.sync_tables()
        h = self.model.hidden_states(ctx)
        logits = self.model.logits(h, want_rows) if want_rows.numel() else None
        for slot, n in zip(ctx.slots, ctx.counts):
            self.cache.advance(slot, n)
        return logits

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
    def decode_step(self, slots: Sequence[int], tokens: Sequence[int], temperature: float = 0.0,
                    top_k: int = 0, top_p: float = 1.0, use_graph: bool = True) -> torch.Tensor:
        """One token for each of ``slots``, then one sampled token each: the
        same kernels as ``step`` + ``sample``, replayed from a CUDA graph that
        is captured the second time a batch size is seen.  Returns the sampled
        tokens as an int32 tensor on the device."""
        from .graph import DecodeGraph
        key = (len(slots), float(temperature), int(top_k), float(top_p))
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = DecodeGraph(self, *key)
        out = g.run(slots, tokens, use_graph)
        self.last_logits = g.last_logits
        return out

    def memory_report(self) -> dict:
        return {"weights_bytes": self.model.weight_bytes(), "cache_bytes": self.cache.bytes(),
                "cache_tokens": self.cache.max_tokens, "slots": self.cache.max_slots}
