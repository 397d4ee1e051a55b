"""The decoder, assembled from a ModelSpec: embedding, blocks run in the
order the schedule gives, final norm and head on the wanted rows.

Nothing here names an architecture.  The reference's counterpart is one
function with per-architecture branches (src/model/layer.rs:1255-1392).
"""

from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..cache.paged import CacheNeed
from ..config.spec import ModelSpec, PartSpec
from ..parts import registry as parts
from ..weights.arena import DictSource, Resident, WeightArena, resident_of
from ..weights.loader import TensorDecl, check_table


def _sub(weights: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorDecl]:
    """Every tensor the model needs, by full name, from the parts' declarations."""
    H, V = spec.hidden_size, spec.vocab_size
    out: Dict[str, TensorDecl] = {}

    def add(prefix: str, decls: Mapping[str, TensorDecl]) -> None:
        for name, d in decls.items():
            out[prefix + name] = d

    add(spec.names["embedding"],
        parts.part_class("embedding", spec.embedding.kind).tensors(spec.embedding.params, H, V))
    for layer in spec.layers:
        add(layer.prefix + layer.names["mixer"],
            parts.part_class("mixer", layer.mixer.kind).tensors(layer.mixer.params, H))
        add(layer.prefix + layer.names["feed_forward"],
            parts.part_class("feed_forward", layer.feed_forward.kind).tensors(
                layer.feed_forward.params, H))
        for site, norm in layer.norms.items():
            add(layer.prefix + layer.names[site],
                parts.part_class("norm", norm.kind).tensors(norm.params, H))
    add(spec.names["final_norm"],
        parts.part_class("norm", spec.final_norm.kind).tensors(spec.final_norm.params, H))
    add(spec.names["head"],
        parts.part_class("head", spec.head.kind).tensors(spec.head.params, H, V))
    return out


def _sites(spec: ModelSpec):
    """(prefix, part class, arguments of its tensors()/resident()) of every part that
    has tensors, in the order the model is built."""
    H, V = spec.hidden_size, spec.vocab_size
    yield (spec.names["embedding"], parts.part_class("embedding", spec.embedding.kind),
           (spec.embedding.params, H, V))
    for layer in spec.layers:
        yield (layer.prefix + layer.names["mixer"], parts.part_class("mixer", layer.mixer.kind),
               (layer.mixer.params, H))
        yield (layer.prefix + layer.names["feed_forward"],
               parts.part_class("feed_forward", layer.feed_forward.kind),
               (layer.feed_forward.params, H))
        for site, norm in layer.norms.items():
            yield (layer.prefix + layer.names[site], parts.part_class("norm", norm.kind),
                   (norm.params, H))
    yield (spec.names["final_norm"], parts.part_class("norm", spec.final_norm.kind),
           (spec.final_norm.params, H))
    yield (spec.names["head"], parts.part_class("head", spec.head.kind), (spec.head.params, H, V))


def resident_plan(spec: ModelSpec) -> Dict[str, Tuple[Resident, str]]:
    """Every tensor the model keeps on the device, by full name, with the prefix of
    the stored tensors it is put together from."""
    plan: Dict[str, Tuple[Resident, str]] = {}
    for prefix, cls, args in _sites(spec):
        for name, res in resident_of(cls, cls.tensors(*args), *args).items():
            plan[prefix + name] = (res, prefix)
    return plan


def place_weights(spec: ModelSpec, source, compute_dtype: torch.dtype, device,
                  where: str = "weights") -> WeightArena:
    """Check ``source``'s tensors against the model's and put them on the device: one
    allocation, every resident tensor written straight to its place."""
    table = source.table()
    if table:
        check_table(where, table, expected_tensors(spec))
    arena = WeightArena(resident_plan(spec), compute_dtype, device,
                        {n: dt for n, (_, dt) in table.items()})
    return arena.fill(source)


class DecoderModel:
    """``weights``: the resident tensors by full name (a :class:`WeightArena`'s
    ``tensors``)."""

    @classmethod
    def from_stored(cls, spec: ModelSpec, stored: Mapping[str, torch.Tensor], rt) -> "DecoderModel":
        """Build from stored tensors held in memory."""
        spec.validate()
        return cls(spec, place_weights(spec, DictSource(stored), rt.dtype, rt.device), rt)

    def __init__(self, spec: ModelSpec, weights, rt):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.arena = weights if isinstance(weights, WeightArena) else None
        if self.arena is not None:
            weights = self.arena.tensors
        H, V = spec.hidden_size, spec.vocab_size
        self.embedding = parts.part_class("embedding", spec.embedding.kind)(
            spec.embedding.params, H, V, _sub(weights, spec.names["embedding"]), rt)
        self.blocks = []
        for layer in spec.layers:
            mixer = parts.part_class("mixer", layer.mixer.kind)(
                layer.mixer.params, H, _sub(weights, layer.prefix + layer.names["mixer"]), rt)
            ff = parts.part_class("feed_forward", layer.feed_forward.kind)(
                layer.feed_forward.params, H,
                _sub(weights, layer.prefix + layer.names["feed_forward"]), rt)
            norms = {site: parts.part_class("norm", n.kind)(
                n.params, H, _sub(weights, layer.prefix + layer.names[site]), rt)
                for site, n in layer.norms.items()}
            self.blocks.append(parts.part_class("block", layer.block)(mixer, ff, norms, rt))
        self.final_norm = parts.part_class("norm", spec.final_norm.kind)(
            spec.final_norm.params, H, _sub(weights, spec.names["final_norm"]), rt)
        self.head = parts.part_class("head", spec.head.kind)(
            spec.head.params, H, V, _sub(weights, spec.names["head"]), rt, self.embedding)

    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """One entry per schedule position; None where the run borrows a cache."""
        needs: List[Optional[CacheNeed]] = []
        for e in self.spec.schedule:
            needs.append(None if e.cache_of is not None
                         else self.blocks[e.layer].mixer.cache_need())
        return needs

    @property
    def captures_prompts(self) -> bool:
        """Whether every part promises that a recorded step of prompts may be replayed for
        other prompts (see StepContext): else prompt steps are launched one by one."""
        # (a run that reads another run's cache reads it by slot, for every row: the rows that
        # fill a recorded step up have none)
        return (getattr(self.embedding, "captures_prompts", False)
                and all(getattr(b, "captures_prompts", False) for b in self.blocks)
                and all(e.cache_of is None for e in self.spec.schedule))

    def hidden_states(self, ctx) -> torch.Tensor:
        """Run every schedule entry over the step's rows; returns the 32-bit
        residual stream [rows, hidden]."""
        rt = self.rt
        if rt.chain_steps and rt.dtype == torch.bfloat16 and 0 < ctx.n_rows <= rt.chain_max_rows:
            # few rows: what lies between two attention kernels runs as one kernel
            with rt.chaining(ctx.n_rows):
                return self._walk(ctx)
        return self._walk(ctx)

    def _walk(self, ctx) -> torch.Tensor:
        from ..parts.base import chain_suspended
        h = self.embedding.forward(ctx)
        schedule = self.spec.schedule
        normed = None
        for pos, e in enumerate(schedule):
            block = self.blocks[e.layer]
            nxt = self.blocks[schedule[pos + 1].layer].first_norm if pos + 1 < len(schedule) else None
            cache_entry = pos if e.cache_of is None else e.cache_of
            if self.rt.chain is not None and not getattr(block, "chain_safe", False):
                with chain_suspended(self.rt):
                    normed = block.forward(h, normed, ctx, pos, cache_entry, e.cache_of is None, nxt)
            else:
                normed = block.forward(h, normed, ctx, pos, cache_entry, e.cache_of is None, nxt)
        return h

    def logits(self, h: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """32-bit logits [len(rows), vocab] of the chosen rows of h."""
        y = self.final_norm.forward(h, out_dtype=self.rt.dtype, rows=rows)
        return self.head.forward(y)

    def weight_bytes(self) -> int:
        """Bytes of the weights a step reads (every resident tensor once)."""
        if self.arena is not None:
            return self.arena.nbytes
        seen, total = set(), 0
        for part in [self.embedding, self.final_norm, self.head] + [
                p for b in self.blocks for p in vars(b).values()]:
            for v in vars(part).values() if hasattr(part, "__dict__") else ():
                if isinstance(v, torch.Tensor) and v.is_cuda:
                    key = v.untyped_storage().data_ptr()
                    if key not in seen:
                        seen.add(key)
                        total += v.untyped_storage().nbytes()
        return total
