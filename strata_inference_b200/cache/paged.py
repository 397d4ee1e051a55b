"""The cache: a slot per sequence, paged keys and values per layer group,
and fixed-size per-sequence state.

* A *slot* belongs to one live sequence and carries its length.  Slots are
  handed back when a sequence ends and are used again without clearing:
  what is valid is known from the length alone, as in the reference
  (src/model/cache.rs:301-310, where ``clear`` only resets the position).
* Keys and values live in *pages* of ``page_tokens`` positions.  Layers
  with the same need (kv heads, head size, window) form a *group* with its
  own pool of pages and its own page table; a sequence's pages are taken
  from the pool as it grows.  A group whose layers see all keys keeps every
  position; a group with a window keeps a ring of the last
  ``ring_tokens`` positions (position p lives in cell p % ring_tokens): the
  window plus room for the longest step that continues a sequence
  (``max_continuation`` positions; by default one page more than the window).
* *State* is a fixed-size tensor per slot and schedule entry for mixers
  that carry a recurrent state instead of keys; it is zeroed when the slot
  is acquired.  (The attention mixer needs none.)

The reference keeps one dense [max_seq_len, kv_dim] buffer per layer and a
single position counter (src/model/cache.rs:23-43,77-112); its errors for
overflow and bad indices (:178-200,218-229) have their counterparts here.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free page (or slot) is left for what a step needs."""


class ContextOverflow(CacheError):
    """A sequence would grow beyond the engine's maximum length."""


@dataclass(frozen=True)
class KVNeed:
    """Per-position keys and values: what an attention-like mixer declares."""

    n_kv_heads: int
    head_dim: int            # width of a key
    window: int = 0          # 0: every earlier position stays visible
    value_dim: int = 0       # width of a value; 0: the same as a key

    @property
    def v_dim(self) -> int:
        return self.value_dim or self.head_dim


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-sequence state: what a recurrent mixer declares."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheNeed:
    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None


class PagePool:
    """Free-list of page numbers with ownership checks."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"{n} pages wanted, {len(self._free)} of {self.n_pages} are free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._held[p]:
                raise CacheError(f"page {p} handed out twice")
            self._held[p] = True
        return out

    def give_back(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages or not self._held[p]:
                raise CacheError(f"page {p} freed but not held")
            self._held[p] = False
            self._free.append(p)


class KVGroup:
    """Storage of the layers (schedule entries) that share one :class:`KVNeed`."""

    def __init__(self, need: KVNeed, entries: List[int], n_pages: int, max_slots: int,
                 max_seq_len: int, page_tokens: int, dtype: torch.dtype, device: torch.device,
                 max_continuation: Optional[int] = None):
        self.need = need
        self.entries = list(entries)
        self.page_tokens = page_tokens
        full_pages = -(-max_seq_len // page_tokens)
        if need.window <= 0:
            ring_pages = full_pages
        elif max_continuation is None:
            ring_pages = -(-need.window // page_tokens) + 1
        else:
            # a step of c positions writes c - 1 cells ahead of what its first row still sees
            ring_pages = -(-(need.window + max(1, max_continuation) - 1) // page_tokens)
        if ring_pages >= full_pages:
            self.ring_tokens = 0          # never wraps
            self.pages_per_seq = full_pages
        else:
            self.ring_tokens = ring_pages * page_tokens
            self.pages_per_seq = ring_pages
        self.n_pages = min(n_pages, max_slots * self.pages_per_seq)
        self.pool = PagePool(self.n_pages)
        shape = (len(entries), self.n_pages, need.n_kv_heads, page_tokens)
        # zeroed once: kernels that work on whole tiles of positions may load a
        # cell that is masked out, and its bits must at least be a number
        self.k = torch.zeros(shape + (need.head_dim,), dtype=dtype, device=device)
        self.v = torch.zeros(shape + (need.v_dim,), dtype=dtype, device=device)
        self.table_host = torch.zeros((max_slots, self.pages_per_seq), dtype=torch.int32)
        self.table = torch.zeros((max_slots, self.pages_per_seq), dtype=torch.int32, device=device)
        self.pages: List[List[int]] = [[] for _ in range(max_slots)]
        self.dirty = False

    def pages_for(self, length: int) -> int:
        """Pages a sequence of ``length`` positions holds in this group."""
        return min(-(-length // self.page_tokens), self.pages_per_seq)

    def max_step_tokens(self, start: Optional[int] = None) -> int:
        """The most positions one step may add to a sequence without overwriting a key
        that a row of the same step still sees: the ring's room beyond the window, which
        holds wherever the sequence stands; a sequence that holds ``start`` positions may
        also add whatever does not wrap around the ring."""
        if self.ring_tokens == 0:
            return 1 << 30
        room = self.ring_tokens - self.need.window + 1
        return room if start is None else max(self.ring_tokens - start, room)

    def bytes(self) -> int:
        return (self.k.numel() + self.v.numel()) * self.k.element_size()


class SequenceCache:
    def __init__(self, needs: Sequence[Optional[CacheNeed]], max_tokens: int, max_seq_len: int,
                 dtype: torch.dtype, device, page_tokens: int = 64,
                 max_slots: Optional[int] = None, max_continuation: Optional[int] = None):
        if page_tokens <= 0 or max_tokens <= 0 or max_seq_len <= 0:
            raise CacheError("page_tokens, max_tokens and max_seq_len must be positive")
        device = torch.device(device)
        self.page_tokens = page_tokens
        self.max_seq_len = max_seq_len
        self.device = device
        self.total_pages = -(-max_tokens // page_tokens)
        self.max_tokens = self.total_pages * page_tokens
        self.max_slots = max_slots or min(self.total_pages, 4096)
        # groups of schedule entries with the same need
        by_need: Dict[KVNeed, List[int]] = {}
        for entry, need in enumerate(needs):
            if need is not None and need.kv is not None:
                by_need.setdefault(need.kv, []).append(entry)
        self.groups: List[KVGroup] = [
            KVGroup(kv, entries, self.total_pages, self.max_slots, max_seq_len, page_tokens,
                    dtype, device, max_continuation) for kv, entries in by_need.items()]
        self._where: Dict[int, Tuple[int, int]] = {}
        for gi, g in enumerate(self.groups):
            for li, entry in enumerate(g.entries):
                self._where[entry] = (gi, li)
        self.state: Dict[int, torch.Tensor] = {}
        for entry, need in enumerate(needs):
            if need is not None and need.state is not None:
                self.state[entry] = torch.zeros((self.max_slots,) + tuple(need.state.shape),
                                                dtype=need.state.dtype, device=device)
        self._free_slots: List[int] = list(range(self.max_slots - 1, -1, -1))
        self._live = [False] * self.max_slots
        self.lengths = [0] * self.max_slots

    # ---- slots --------------------------------------------------------
    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def acquire(self) -> int:
        if not self._free_slots:
            raise CacheFull(f"all {self.max_slots} slots are in use")
        s = self._free_slots.pop()
        if self._live[s]:
            raise CacheError(f"slot {s} handed out twice")
        self._live[s] = True
        self.lengths[s] = 0
        for t in self.state.values():
            t[s].zero_()
        return s

    def release(self, slot: int) -> None:
        self._check_slot(slot)
        for g in self.groups:
            g.pool.give_back(g.pages[slot])
            g.pages[slot] = []
        self._live[slot] = False
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    def _check_slot(self, slot: int) -> None:
        if not isinstance(slot, int) or not 0 <= slot < self.max_slots:
            raise CacheError(f"slot {slot!r} does not exist (0..{self.max_slots - 1})")
        if not self._live[slot]:
            raise CacheError(f"slot {slot} is not in use")

    def length(self, slot: int) -> int:
        self._check_slot(slot)
        return self.lengths[slot]

    def live_slots(self) -> List[int]:
        return [s for s, l in enumerate(self._live) if l]

    # ---- growth -------------------------------------------------------
    def reserve(self, grow: Sequence[Tuple[int, int]]) -> None:
        """Make room for ``n`` more positions in each ``(slot, n)``; either
        every sequence gets its pages or nothing changes."""
        plan = []
        wanted = [0] * len(self.groups)
        for slot, n in grow:
            self._check_slot(slot)
            new_len = self.lengths[slot] + n
            if n < 0 or new_len > self.max_seq_len:
                raise ContextOverflow(f"slot {slot}: {self.lengths[slot]} + {n} positions exceed "
                                      f"the maximum sequence length {self.max_seq_len}")
            for gi, g in enumerate(self.groups):
                extra = g.pages_for(new_len) - len(g.pages[slot])
                if extra > 0:
                    plan.append((gi, slot, extra))
                    wanted[gi] += extra
        for gi, g in enumerate(self.groups):
            if wanted[gi] > g.pool.n_free:
                raise CacheFull(f"the cache holds {self.max_tokens} positions; {wanted[gi]} more "
                                f"pages of {self.page_tokens} are needed and {g.pool.n_free} are free")
        for gi, slot, extra in plan:
            g = self.groups[gi]
            have = len(g.pages[slot])
            new = g.pool.take(extra)
            g.pages[slot].extend(new)
            g.table_host[slot, have:have + extra] = torch.tensor(new, dtype=torch.int32)
            g.dirty = True

    def advance(self, slot: int, n: int) -> None:
        self._check_slot(slot)
        self.lengths[slot] += n

    def trim(self, slot: int) -> None:
        """Give back the pages ``slot`` holds beyond what its length needs (what a step
        reserved and then did not use because it failed)."""
        self._check_slot(slot)
        for g in self.groups:
            keep = g.pages_for(self.lengths[slot])
            extra = g.pages[slot][keep:]
            if extra:
                g.pool.give_back(extra)
                del g.pages[slot][keep:]

    def sync_tables(self) -> None:
        """Bring the device copies of changed page tables up to date."""
        for g in self.groups:
            if g.dirty:
                g.table.copy_(g.table_host, non_blocking=True)
                g.dirty = False

    def max_step_tokens(self, start: Optional[int] = None) -> int:
        """The most positions a step may add to a sequence (that holds ``start`` positions)."""
        return min([g.max_step_tokens(start) for g in self.groups] or [1 << 30])

    # ---- views --------------------------------------------------------
    def kv_view(self, entry: int) -> "KVView":
        gi, li = self._where[entry]
        g = self.groups[gi]
        return KVView(g.k[li], g.v[li], g.table, g.page_tokens, g.ring_tokens, g.need)

    def has_kv(self, entry: int) -> bool:
        return entry in self._where

    def state_view(self, entry: int) -> torch.Tensor:
        return self.state[entry]

    def pages_in_use(self) -> int:
        return sum(g.n_pages - g.pool.n_free for g in self.groups)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups)


@dataclass
class KVView:
    """What a mixer sees of one schedule entry's keys and values."""

    k: torch.Tensor            # [pages, kv_heads, page_tokens, head_dim]
    v: torch.Tensor            # [pages, kv_heads, page_tokens, value_dim]
    page_table: torch.Tensor   # [slots, pages_per_seq] int32, on the device
    page_tokens: int
    ring_tokens: int           # 0: position p lives in cell p
    need: KVNeed
