"""The attention mixer: grouped-query attention over the paged cache.

Parameters (all from the PartSpec): ``num_heads``, ``num_kv_heads``,
``head_dim`` (heads x head_dim need not equal the hidden size),
``score_scale`` (the factor on q.k), ``logit_softcap`` (0: off), ``window``
(0: every earlier key is visible; W: the last W keys, the query's own
included) and ``position`` (a PartSpec of a position encoding).

Order of operations, as in the reference (src/model/layer.rs:1113-1161,
872-984): q, k, v projections (no bias); rotation of q and k; k and v
appended to the cache at the rows' positions; scores scaled, soft-capped,
masked; softmax; weighted sum of v; output projection.

A step whose sequences all begin at position 0 (prompts) attends over the
step's own k and v rows; any other step attends over the cache.  A run that
borrows another schedule entry's cache projects q only and reads that cache.

Fast paths inside this general part (each falls back to the general kernels
when its condition does not hold, with the same result): for at most 16
bfloat16 rows, a position part that offers ``rotary()`` with half-split pairs
over the WHOLE head lets the q|k|v product rotate and store in its own
epilogue (partial rotary or interleaved pairs take the product and then the
rotate-and-store kernel); prompts take the tcgen05 attention for head sizes
64/128/256 with at most two query heads per kv head, else the mma.sync
kernel, else the general one; single rows over the cache take the
bandwidth-tuned kernel for head sizes 64/128/256 and groups of 1, 2, 4 or 8.
"""

from __future__ import annotations

import os
from typing import Dict, Mapping, Optional

import torch

from ..cache.paged import CacheNeed, KVNeed
from ..config.spec import ConfigError, PartSpec
from ..kernels import native
from ..weights.arena import Piece, Resident, resident_of
from ..weights.loader import TensorDecl
from .registry import part_class, register_mixer

# warps per SM of the general attention kernel that a split of the keys aims at
_WARPS_PER_SM = 16
# SIB_PREFILL_TCGEN05=0 selects the mma.sync prompt kernel instead of the tcgen05 one
_USE_TCGEN05_PREFILL = os.environ.get("SIB_PREFILL_TCGEN05", "1") != "0"


def decode_shape(units: int, longest: int, window: int, resident4: int, resident8: int,
                 block_warps=(8, 4, 2)):
    """(runs, warps) of the decode kernel for ``units`` (row, kv head) pairs whose rows see up
    to ``longest`` keys, on a device that holds ``resident4`` warps of the kernel in blocks of
    4 (or fewer) warps and ``resident8`` in blocks of 8 (``Attention._decode_shape`` says why)."""
    # (a full window does not begin at a tile's first key: it reaches into one tile more)
    tiles = -(-longest // 16) + (1 if 0 < window <= longest else 0)

    def fewest(resident: int) -> int:
        """Warps for a (row, kv head): as few tiles each as ``resident`` warps allow."""
        room = max(1, resident // units)
        each = -(-tiles // room)
        return max(1, min(room, -(-tiles // each)))

    def trimmed(runs: int, warps: int):
        """Without the blocks that whole blocks of ``warps`` warps leave no tile for."""
        each = -(-tiles // (runs * warps))
        return -(-(-(-tiles // each)) // warps), warps

    most = fewest(resident4)
    if 8 in block_warps and resident8 // units >= 8:
        wide = min(-(-fewest(resident8) // 8), resident8 // units // 8, 128)
        if wide >= 8 and 8 * wide >= 0.6 * most:
            return trimmed(wide, 8)
    room = max(1, resident4 // units)
    for warps in (w for w in block_warps if w < 8):   # wider blocks: fewer results to join
        runs = min(-(-most // warps), room // warps, 128)
        if runs >= 1 and runs * warps >= 0.9 * most:
            return trimmed(runs, warps)
    return trimmed(min(most, 128), 1)


class Attention:
    chain_safe = True      # deferred results are read by this runtime's and native's launchers only

    @property
    def captures_prompts(self) -> bool:
        """Whether a step of prompts of this part may be recorded and replayed for other
        prompts (StepContext ``from_start``): it then reads sequences, slots and counts on
        the device only.  True with a rotary position part, or one that promises the same."""
        return hasattr(self.position, "rotary") or getattr(self.position, "captures_prompts", False)

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        nh, nkv, hd = params["num_heads"], params["num_kv_heads"], params["head_dim"]
        out = {
            "q_proj.weight": TensorDecl((nh * hd, hidden)),
            "k_proj.weight": TensorDecl((nkv * hd, hidden)),
            "v_proj.weight": TensorDecl((nkv * hd, hidden)),
            "o_proj.weight": TensorDecl((hidden, nh * hd)),
        }
        pos: PartSpec = params["position"]
        for name, decl in part_class("position", pos.kind).tensors(pos.params, hd).items():
            out["position." + name] = decl
        return out

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        """q, k and v are kept as ONE matrix (one product makes all three)."""
        nh, nkv, hd = params["num_heads"], params["num_kv_heads"], params["head_dim"]
        out = {
            "qkv_proj.weight": Resident(((nh + 2 * nkv) * hd, hidden), pieces=(
                Piece("q_proj.weight", 0), Piece("k_proj.weight", nh * hd),
                Piece("v_proj.weight", (nh + nkv) * hd))),
            "o_proj.weight": Resident((hidden, nh * hd), pieces=(Piece("o_proj.weight"),)),
        }
        pos: PartSpec = params["position"]
        cls = part_class("position", pos.kind)
        for name, res in resident_of(cls, cls.tensors(pos.params, hd), pos.params, hd).items():
            out["position." + name] = Resident(res.shape, res.dtype, tuple(
                Piece("position." + q.source, q.row_offset, q.group, q.group_stride)
                for q in res.pieces), res.offset)
        return out

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.rt = rt
        self.hidden = hidden
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.hd = int(params["head_dim"])
        self.scale = float(params["score_scale"])
        self.softcap = float(params.get("logit_softcap") or 0.0)
        self.window = int(params.get("window") or 0)
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"attention: {self.nh} heads cannot share {self.nkv} kv heads")
        if self.hd % 16 or not 16 <= self.hd <= 512:
            raise ConfigError(f"attention: head_dim {self.hd} must be a multiple of 16 "
                              f"between 16 and 512")
        pos: PartSpec = params["position"]
        pos_w = {k[len("position."):]: v for k, v in weights.items() if k.startswith("position.")}
        self.position = part_class("position", pos.kind)(pos.params, self.hd, pos_w, rt)
        self.w_qkv = rt.cast_matrix(weights["qkv_proj.weight"])
        self.w_q = self.w_qkv[: self.nh * self.hd]
        self.w_o = rt.cast_matrix(weights["o_proj.weight"])
        self._resident_warps: Optional[int] = None
        self._target_warps = _WARPS_PER_SM * rt.sm_count
        self._block_warps = tuple(int(w) for w in os.environ.get("SIB_DECODE_WARPS", "8,4,2").split(","))

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(kv=KVNeed(self.nkv, self.hd, self.window))

    # ------------------------------------------------------------------
    def _longest(self, ctx, capacity: int) -> int:
        longest = (min(ctx.span or capacity, capacity)) if ctx.graph_capture else ctx.max_end
        return min(longest, self.window) if self.window > 0 else longest

    def _splits(self, ctx, capacity: int) -> int:
        """How many runs of keys the general kernel cuts a (row, head) into, one
        warp each: as many as fill the device once, none shorter than 32 keys."""
        want = max(1, self._target_warps // max(1, ctx.n_rows * self.nh))
        return max(1, min(want, -(-self._longest(ctx, capacity) // 32), 128))

    def _decode_shape(self, ctx, capacity: int):
        """(runs, warps) for the decode kernel: each (row, kv head) is read by
        ``runs`` blocks of ``warps`` warps.  All of them should be resident at
        once (a second, partly filled wave of blocks costs more than it brings).  A warp
        walks its tiles of 16 keys one after the other, a round trip to memory each, so a
        (row, kv head) gets as many warps as give each the fewest tiles that residency
        allows, and no more than that needs: more warps only mean more partial results to
        join.  (Before, a warp took no fewer than 32 keys and all the warps that fit: with the
        rule above batch 1 went from 1.64 to 1.57 ms at context 1 024 and from 1.72 to 1.68 ms at
        8 192, batch 16 from 2.07 to 1.98 ms at context 1 024; no size measured lost, on the 9B
        and 27B shapes neither.)  Blocks of 8 warps (of which the device holds fewer warps in all) halve the
        partial results that the last block of a (row, kv head) joins: they are taken where
        that join weighs most, with few rows and therefore many runs each (measured at the
        Gemma2-2B shape, context 8 192: batch 1 1.83 -> 1.74 ms, batch 2 1.95 -> 1.84, batch 4
        2.06 -> 2.04; batch 6 and 8 are better off with blocks of 4)."""
        if self._resident_warps is None:     # what the device holds of this kernel at a time
            self._resident_warps = {w: native.attention_decode_resident_warps(self.nh, self.nkv, self.hd, w)
                                    for w in (8, 4)}
        return decode_shape(max(1, ctx.n_rows * self.nkv), self._longest(ctx, capacity), self.window,
                            self._resident_warps[4], self._resident_warps[8], self._block_warps)

    def _pieces_pay(self, ctx) -> bool:
        """Whether copying what the step's sequences hold (read, write, read again by the
        prompt kernel) moves less than reading it row by row does."""
        seen = float(self.window) if self.window > 0 else float("inf")
        by_row = sum(n * min(seen, st + n / 2) for st, n in zip(ctx.starts, ctx.counts))
        copied = sum(min(seen + n, st + n) for st, n in zip(ctx.starts, ctx.counts))
        return by_row > 3 * copied

    def _attend_pieces(self, qkv: torch.Tensor, out: torch.Tensor, ctx, view) -> None:
        """Attention of a step that continues sequences with many tokens each (a prompt that
        comes in pieces): the keys and values that the rows see - what the sequences held and
        what this step has just stored - are copied from the pages into a packed buffer
        whose rows are positions, the step's queries are put at their positions, and the
        prompt kernel runs over it with the rows before each piece as keys only.  (Row by row
        over the cache, as single-token steps do it, every row reads its sequence's whole
        past: 4 096 tokens in pieces of 512 took 183 ms instead of 15 ms in one piece.)"""
        rt, nh, nkv, hd = self.rt, self.nh, self.nkv, self.hd
        memo = ctx.memo.setdefault(("pieces", self.window), {})
        if not memo:
            starts, counts = ctx.starts, ctx.counts
            ends = [st + n for st, n in zip(starts, counts)]
            first = [max(0, st - self.window + 1) if self.window > 0 else 0 for st in starts]
            row0, acc = [], 0
            for e in ends:
                row0.append(acc)
                acc += e
            dev = lambda v: torch.tensor(v, dtype=torch.int32).to(qkv.device, non_blocking=True)  # noqa: E731
            memo.update(row0=row0, ends=ends, first=first, rows=acc, d_row0=dev(row0), d_ends=dev(ends),
                        d_first=dev(first), d_starts=dev(starts),
                        most=max(e - f for e, f in zip(ends, first)))
            memo["plan"] = native.attention_prefill_tc_plan(ends, nh, nkv, hd, self.window, starts)
        width = (nh + 2 * nkv) * hd
        # (one packed buffer and one output buffer a step: the layers use them in turn)
        shared = ctx.memo.setdefault(("pieces", "buffers", width, nh * hd), {})
        if not shared:
            # (zeros: a windowed layer copies only what its rows see, but the kernel's key
            # tiles reach further down and over a sequence's end into the next one's rows;
            # what is masked there must still be finite, or 0 x NaN spoils the sums)
            shared["packed"] = torch.zeros((memo["rows"], width), dtype=qkv.dtype, device=qkv.device)
            shared["whole"] = torch.empty((memo["rows"], nh * hd), dtype=qkv.dtype, device=qkv.device)
        packed, whole = shared["packed"], shared["whole"]
        native.gather_kv_rows(packed, view.k, view.v, view.page_table, ctx.seq_slot, memo["d_first"],
                              memo["d_ends"], memo["d_row0"], memo["most"], view.page_tokens,
                              view.ring_tokens, nh, nkv, hd)
        r = 0
        for row0, st, n in zip(memo["row0"], ctx.starts, ctx.counts):
            packed[row0 + st:row0 + st + n, :nh * hd].copy_(qkv[r:r + n, :nh * hd])
            r += n
        n_items, need, n_tickets = memo["plan"]
        lens = memo["ends"] if n_items else None
        if not n_items:
            need, n_tickets = native.attention_prefill_tc_split(ctx.n_seqs, max(memo["ends"]), nh, nkv, hd)
        native.attention_prefill_tc(packed, whole, memo["d_row0"], memo["d_ends"], ctx.n_seqs,
                                    max(memo["ends"]), nh, nkv, hd, self.scale, self.softcap,
                                    self.window, rt.scratch(need) if need else None,
                                    rt.tickets(n_tickets) if need else None, lens,
                                    memo["d_starts"], ctx.starts if lens else None)
        r = 0
        for row0, st, n in zip(memo["row0"], ctx.starts, ctx.counts):
            out[r:r + n].copy_(whole[row0 + st:row0 + st + n])
            r += n

    def forward(self, x: torch.Tensor, ctx, entry: int, cache_entry: int,
                owns_cache: bool) -> torch.Tensor:
        rt, nh, hd = self.rt, self.nh, self.hd
        R = x.shape[0]
        nkv = self.nkv if owns_cache else 0
        view = ctx.kv(cache_entry)
        fresh = ctx.all_from_start and owns_cache
        if not fresh and view.ring_tokens > 0 and not ctx.graph_capture:
            # rows that attend over a ring must not overwrite a key that an earlier row of
            # the same step still sees (a captured step adds one position: always fine)
            room = view.ring_tokens - self.window + 1
            for start, n in zip(ctx.starts, ctx.counts):
                if n > room and start + n > view.ring_tokens:
                    raise ValueError(
                        f"a step may add at most {max(room, view.ring_tokens - start)} positions "
                        f"to a sequence of {start} whose layers keep a window of {self.window} "
                        f"in a ring of {view.ring_tokens}; got {n}")

        w_in = self.w_qkv if owns_cache else self.w_q
        rotary = self.position.rotary() if hasattr(self.position, "rotary") else None
        if (rotary is not None and rotary[1] == hd and rotary[2] == native.ROPE_HALF_SPLIT
                and x.dtype == torch.bfloat16 and rt.fuse_rotation and 0 < R <= rt.fused_rope_max_rows
                and self.hidden % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0):
            # few rows: the product rotates q and k and writes k and v into the cache itself
            qkv = torch.empty((R, w_in.shape[0]), dtype=x.dtype, device=x.device)
            rt.linear_rope(x, w_in, qkv, row_pos=ctx.row_pos, row_seq=ctx.row_seq,
                           seq_slot=ctx.seq_slot, seq_end=ctx.seq_end, inv_freq=rotary[0],
                           k_pool=view.k if owns_cache else None,
                           v_pool=view.v if owns_cache else None,
                           page_table=view.page_table if owns_cache else None,
                           page_tokens=view.page_tokens, ring_tokens=view.ring_tokens,
                           n_heads=nh, n_kv=nkv, head_dim=hd)
        else:
            qkv = rt.linear(x, w_in)
            if rotary is not None:
                inv_freq, rot, style = rotary
            else:
                rt.flush()      # a position part of its own works on q and k with its own code
                q_view = qkv[:, : nh * hd].view(R, nh, hd)
                k_view = qkv[:, nh * hd:(nh + nkv) * hd].view(R, nkv, hd) if nkv else None
                self.position.apply(q_view, k_view, ctx)
                inv_freq, rot, style = None, 0, native.ROPE_HALF_SPLIT
            native.rope_store(qkv, ctx.row_pos, ctx.row_seq, ctx.seq_slot, ctx.seq_end, inv_freq,
                              rot, style, view.k if owns_cache else None,
                              view.v if owns_cache else None,
                              view.page_table if owns_cache else None, view.page_tokens,
                              view.ring_tokens, nh, nkv, hd)

        out = torch.empty((R, nh * hd), dtype=qkv.dtype, device=qkv.device)
        width = qkv.shape[1]
        # (prompts of up to 128 tokens: the mma.sync kernel, whose blocks of 64 rows start in a
        # fraction of the time that a tcgen05 block needs before its first tile; measured on 2 048
        # rows of the Gemma2-2B shape: 64 prompts of 32 tokens 22 against 65 us a call, 16 of 128
        # 28 against 39 us, 8 of 256 36 against 56 us the other way round)
        short = ctx.max_count <= rt.short_prompt_tokens and native.attention_prefill_supports(
            nh, self.nkv, hd)
        if fresh and qkv.dtype == torch.bfloat16 and _USE_TCGEN05_PREFILL and self.scale > 0 and \
                not short and native.attention_prefill_tc_supports(nh, self.nkv, hd, width):
            # a launch too small for the device splits its long blocks, given the memory
            # (with the lengths known on the host, not in a recorded step, the launch is a
            # balanced list of work items)
            lens = None if ctx.graph_capture else ctx.counts
            n_items = 0
            if lens is not None:
                n_items, need, n_tickets = native.attention_prefill_tc_plan(lens, nh, self.nkv, hd,
                                                                            self.window)
            if n_items == 0:
                lens = None
                need, n_tickets = native.attention_prefill_tc_split(ctx.n_seqs, ctx.max_count, nh,
                                                                   self.nkv, hd)
            native.attention_prefill_tc(qkv, out, ctx.seq_row0, ctx.seq_end, ctx.n_seqs,
                                        ctx.max_count, nh, self.nkv, hd, self.scale, self.softcap,
                                        self.window, rt.scratch(need) if need else None,
                                        rt.tickets(n_tickets) if need else None, lens)
        elif fresh and qkv.dtype == torch.bfloat16 and \
                native.attention_prefill_supports(nh, self.nkv, hd):
            native.attention_prefill(qkv, out, ctx.seq_row0, ctx.seq_end, ctx.n_seqs,
                                     ctx.max_count, nh, self.nkv, hd, self.scale, self.softcap,
                                     self.window)
        elif fresh:
            k_new = qkv[:, nh * hd:]
            v_new = qkv[:, (nh + nkv) * hd:]
            native.attention_rows(qkv, width, k_new, v_new, width, None, None, None,
                                  view.page_tokens, view.ring_tokens, ctx.row_pos, ctx.row_seq,
                                  ctx.seq_slot, ctx.seq_start, ctx.seq_row0, out, None, nh,
                                  self.nkv, hd, self.scale, self.softcap, self.window, 1)
        elif (qkv.dtype == torch.bfloat16 and not ctx.graph_capture
              and ctx.max_count >= rt.piece_attention_rows and _USE_TCGEN05_PREFILL and self.scale > 0
              and native.attention_prefill_tc_supports(nh, self.nkv, hd, (nh + 2 * self.nkv) * hd)
              and self._pieces_pay(ctx)):
            self._attend_pieces(qkv, out, ctx, view)
        elif qkv.dtype == torch.bfloat16 and native.attention_decode_supports(
                nh, self.nkv, hd, view.page_tokens):
            splits, warps = self._decode_shape(ctx, ctx.cache.max_seq_len)
            scratch = tickets = None
            if splits > 1:
                scratch = rt.scratch(native.attention_rows_scratch_bytes(R, nh, hd, splits))
                tickets = rt.tickets(R * self.nkv)
            native.attention_decode(qkv, width, view.k, view.v, view.page_table, view.page_tokens,
                                    view.ring_tokens, ctx.row_pos, ctx.row_seq, ctx.seq_slot, out,
                                    scratch, tickets, nh, self.nkv, hd, self.scale, self.softcap,
                                    self.window, splits, warps,
                                    fresh=ctx.max_count if rt.early_keys else 0)
        else:
            splits = self._splits(ctx, ctx.cache.max_seq_len)
            scratch = None
            if splits > 1:
                scratch = rt.scratch(native.attention_rows_scratch_bytes(R, nh, hd, splits))
            native.attention_rows(qkv, width, None, None, width, view.k, view.v, view.page_table,
                                  view.page_tokens, view.ring_tokens, ctx.row_pos, ctx.row_seq,
                                  ctx.seq_slot, ctx.seq_start, ctx.seq_row0, out, scratch, nh,
                                  self.nkv, hd, self.scale, self.softcap, self.window, splits)
        return rt.linear(out, self.w_o)


register_mixer("attention", Attention)
