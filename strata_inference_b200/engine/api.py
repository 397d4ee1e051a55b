"""The Python entry point, in the reference's manner.

The reference's ``GenerationEngine`` (src/engine/generate.rs:154-235,
588-632, 1140-1177) owns configuration, weights and executor, and offers
``generate*`` methods that take a ``GenerationConfig``; its
``generate_from_token_ids`` bypasses the tokenizer.  This library works on
token ids only (it has no tokenizer), takes batches, and loads a model
folder (config.json + safetensors) instead of a GGUF file:

    engine = GenerationEngine.from_dir("model_dir", dtype="bfloat16")
    outs = engine.generate([[2, 17, 5], [2, 9]], GenerationConfig(max_tokens=16))
    outs[0].token_ids, outs[0].stop_reason
"""

from __future__ import annotations

from typing import Callable, List, Mapping, Optional, Sequence

import torch

from ..sampling.sampler import SamplingConfig
from .engine import Engine
from .generate import GenerationConfig, GenerationOutput, generate


class EngineStepper:
    """What the generation loop needs of an :class:`Engine`."""

    def __init__(self, engine: Engine, use_graph: bool = True):
        self.engine = engine
        self.use_graph = use_graph
        self.max_seq_len = engine.max_seq_len
        self.page_tokens = engine.cache.page_tokens
        self.default_stop_tokens = tuple(engine.spec.stop_tokens)

    @property
    def capacity_tokens(self) -> int:
        """Positions the cache can still take (the groups that keep every
        position decide; a model without keys is bounded by its slots only)."""
        groups = self.engine.cache.groups
        if not groups:
            return self.engine.cache.max_tokens
        full = [g.pool.n_free for g in groups if g.ring_tokens == 0]
        free = min(full) if full else min(g.pool.n_free for g in groups)
        return free * self.page_tokens

    @property
    def free_slots(self) -> int:
        return self.engine.cache.n_free_slots

    def new_sequence(self) -> int:
        return self.engine.new_sequence()

    def end_sequence(self, slot: int) -> None:
        self.engine.end_sequence(slot)

    def length(self, slot: int) -> int:
        return self.engine.length(slot)

    def seed(self, slot: int, seed: int) -> None:
        self.engine.seed_sequence(slot, seed)

    def prefill(self, slots, prompts, sampling: SamplingConfig) -> List[int]:
        logits = self.engine.step(list(zip(slots, prompts)))
        self.engine.last_logits = logits
        toks = self.engine.sample(logits, slots, sampling.temperature, sampling.top_k,
                                  sampling.top_p)
        return self.engine.read_back(toks)

    def decode(self, slots, tokens, sampling: SamplingConfig) -> List[int]:
        return self.decode_collect(self.decode_issue(slots, tokens, sampling))

    # The same in two halves, so that the loop can issue the step after this one before it
    # reads this one's tokens (the device then never waits for the host between steps):
    def decode_issue(self, slots, tokens, sampling: SamplingConfig):
        """Launch the step; ``tokens`` None: the ones the step before sampled for the same
        slots (``can_feed_back``).  Returns a ticket for ``decode_collect``."""
        out = self.engine.decode_step(slots, tokens, sampling.temperature, sampling.top_k,
                                      sampling.top_p, use_graph=self.use_graph)
        return self.engine.read_later(out)

    def decode_collect(self, ticket) -> List[int]:
        return self.engine.read_now(ticket)

    def can_feed_back(self, slots, sampling: SamplingConfig) -> bool:
        return self.use_graph and self.engine.can_feed_back(
            slots, sampling.temperature, sampling.top_k, sampling.top_p)


class GenerationEngine:
    def __init__(self, engine: Engine, use_graph: bool = True):
        self.engine = engine
        self._stepper = EngineStepper(engine, use_graph)

    @classmethod
    def from_dir(cls, model_dir: str, dtype="bfloat16", ctx: Optional[int] = None,
                 max_tokens: int = 8192, use_graph: bool = True, **kw) -> "GenerationEngine":
        """``ctx`` lowers the maximum sequence length (the reference's ``--ctx``,
        src/engine/generate.rs:252-256); ``max_tokens`` sizes the cache."""
        return cls(Engine.from_dir(model_dir, dtype, max_tokens=max_tokens, max_seq_len=ctx, **kw),
                   use_graph)

    @classmethod
    def from_random(cls, config: Mapping, seed: int, dtype="bfloat16",
                    ctx: Optional[int] = None, max_tokens: int = 8192, use_graph: bool = True,
                    **kw) -> "GenerationEngine":
        return cls(Engine.from_random(config, seed, dtype, max_tokens=max_tokens,
                                      max_seq_len=ctx, **kw), use_graph)

    def last_logits(self) -> Optional[torch.Tensor]:
        """32-bit logits [sequences, vocab] the latest tokens were sampled from
        (valid until the next step)."""
        return self.engine.last_logits

    @property
    def vocab_size(self) -> int:
        return self.engine.vocab_size

    @property
    def max_seq_len(self) -> int:
        return self.engine.max_seq_len

    def generate(self, prompts: Sequence[Sequence[int]],
                 config: Optional[GenerationConfig] = None,
                 callback: Optional[Callable[[int, int], bool]] = None,
                 seeds: Optional[Sequence[int]] = None) -> List[GenerationOutput]:
        """Generate for a batch of token-id prompts (see engine/generate.py)."""
        return generate(self._stepper, prompts, config or GenerationConfig(), callback, seeds)

    def generate_from_token_ids(self, token_ids: Sequence[int],
                                config: Optional[GenerationConfig] = None,
                                callback: Optional[Callable[[int], bool]] = None
                                ) -> GenerationOutput:
        """One request (src/engine/generate.rs:1140-1177)."""
        cb = None if callback is None else (lambda _i, t: callback(t))
        return self.generate([token_ids], config, cb)[0]
