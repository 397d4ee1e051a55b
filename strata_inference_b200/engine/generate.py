"""The generation loop: batches of unequal prompts, stop tokens, sequences
that end earlier, one batch after another until every request is served.

Per sequence the decisions are the reference's, in its order
(src/engine/generate.rs:655-778):

* an empty prompt and a prompt of ``max_seq_len`` tokens or more are errors;
* the whole prompt is one step; its last row's logits give the first token;
* then, up to ``max_tokens`` times: a stop token ends the sequence and is
  not emitted ("eos"); otherwise the token is emitted and streamed; a
  callback that returns False ends it ("cancelled", the token is kept); a
  full context ends it ("context_length", the token is kept but never fed);
  otherwise the token is fed as a one-token step and the next one sampled;
* running out of ``max_tokens`` ends it ("max_tokens").

A batch's requests start together; a finished sequence leaves the batch and
gives its slot back at once; the next batch starts when the current one is
done.  The loop talks to the model through a small *stepper* (prefill,
decode, slots), so its decisions can be tested without a device.

Looking ahead.  Reading a step's tokens, deciding and launching the next step leaves the
device idle for as long as the host takes.  A stepper that can launch a step and hand out
its tokens later (``decode_issue`` / ``decode_collect``) and can feed a step with the
tokens the step before sampled, on the device (``can_feed_back``), is therefore kept one
step ahead: while the host reads and judges the tokens of step n, step n + 1 is already
running for the same sequences.  If a sequence ends at step n, its row of step n + 1 is
dropped unseen and the others' rows are kept; every decision and every emitted token is
the same as without looking ahead.  A sequence is never fed beyond the context's end,
and no step is launched that no sequence could use.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling.sampler import SamplingConfig

STOP_TOKEN = "eos"
MAX_TOKENS = "max_tokens"
CONTEXT_LENGTH = "context_length"
CANCELLED = "cancelled"


class GenerationError(ValueError):
    pass


@dataclass
class GenerationConfig:
    """src/engine/generate.rs:86-104.  ``max_tokens`` < 0: until a stop token or the context's end."""

    max_tokens: int = 256
    stop_tokens: Sequence[int] = ()
    sampling: SamplingConfig = field(default_factory=SamplingConfig)
    # Keep the device one step ahead of the host (see the module's text).  The logits that
    # a stepper shows for "the latest step" are then those of a later step than the token a
    # callback is looking at: switch it off to read them token by token.
    look_ahead: bool = True


@dataclass
class GenerationOutput:
    """src/engine/generate.rs:73-83, plus the time spent decoding."""

    token_ids: List[int]
    stop_reason: str
    prompt_tokens: int
    prefill_duration: float
    decode_duration: float = 0.0


def _round_up(n: int, unit: int) -> int:
    return -(-n // unit) * unit


def plan_batch(lengths: Sequence[int], max_tokens: int, max_seq_len: int, page_tokens: int,
               capacity_tokens: int, free_slots: int) -> int:
    """How many of the waiting requests (in order) start together: as many as
    the cache can hold to their ends.  At least one, or an error."""
    used, n = 0, 0
    for length in lengths:
        end = max_seq_len if max_tokens < 0 else min(length + max_tokens, max_seq_len)
        need = _round_up(max(end, length), page_tokens)
        if n >= free_slots or used + need > capacity_tokens:
            break
        used += need
        n += 1
    if n == 0:
        raise GenerationError(
            f"a request of {lengths[0]} prompt tokens and up to "
            f"{'the context end' if max_tokens < 0 else max_tokens} new tokens does not fit "
            f"the cache ({capacity_tokens} positions, {free_slots} free slots)")
    return n


def generate(stepper, prompts: Sequence[Sequence[int]], config: GenerationConfig,
             callback: Optional[Callable[[int, int], bool]] = None,
             seeds: Optional[Sequence[int]] = None) -> List[GenerationOutput]:
    """Generate for every prompt.  ``callback(request_index, token)`` is called
    for every emitted token; returning False cancels that request.  Every
    request draws from its own generator, seeded with ``seeds[i]`` if given,
    else with the configured seed: a request samples the same tokens alone or
    in any batch."""
    if not prompts:
        return []
    max_seq_len = stepper.max_seq_len
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise GenerationError(f"request {i}: empty prompt")
        if len(p) >= max_seq_len:
            raise GenerationError(f"request {i}: prompt length ({len(p)}) exceeds "
                                  f"max_seq_len ({max_seq_len})")
    if seeds is not None and len(seeds) != len(prompts):
        raise GenerationError("'seeds' needs one seed per prompt")
    stops = set(int(t) for t in config.stop_tokens) | set(stepper.default_stop_tokens)
    limit = config.max_tokens
    results: List[Optional[GenerationOutput]] = [None] * len(prompts)
    waiting = list(range(len(prompts)))

    while waiting:
        n = plan_batch([len(prompts[i]) for i in waiting], limit, max_seq_len,
                       stepper.page_tokens, stepper.capacity_tokens, stepper.free_slots)
        batch, waiting = waiting[:n], waiting[n:]
        held = set()
        live = []
        try:
            slots = []
            for _ in batch:
                slots.append(stepper.new_sequence())
                held.add(slots[-1])
            for i, s in zip(batch, slots):
                stepper.seed(s, seeds[i] if seeds is not None else config.sampling.seed_value())
            t0 = time.perf_counter()
            nxt = stepper.prefill(slots, [prompts[i] for i in batch], config.sampling)
            prefill_s = time.perf_counter() - t0
            for i, s, t in zip(batch, slots, nxt):
                results[i] = GenerationOutput([], MAX_TOKENS, len(prompts[i]), prefill_s)
                live.append((i, s, int(t)))
            t_decode = time.perf_counter()
            # a stepper without the two halves: the ticket of a step is its tokens
            issue = getattr(stepper, "decode_issue", None) or stepper.decode
            collect = getattr(stepper, "decode_collect", None) or (lambda ticket: ticket)
            ahead_ok = config.look_ahead and hasattr(stepper, "decode_issue")
            ahead = None        # ticket of a step already running for the sequences of `live`
            while live:
                going = []
                for i, s, tok in live:
                    out = results[i]
                    reason = None
                    if limit >= 0 and len(out.token_ids) >= limit:
                        reason = MAX_TOKENS
                    elif tok in stops:
                        reason = STOP_TOKEN
                    else:
                        out.token_ids.append(tok)
                        if callback is not None and not callback(i, tok):
                            reason = CANCELLED
                        elif out.prompt_tokens + len(out.token_ids) - 1 >= max_seq_len:
                            # (the positions the cache holds once every emitted token but
                            # this one is fed: the context is full)
                            reason = CONTEXT_LENGTH
                        elif limit >= 0 and len(out.token_ids) >= limit:
                            # the reference runs one more step here and drops its
                            # token; the outcome is the same without the step
                            reason = MAX_TOKENS
                    if reason is None:
                        going.append((i, s, tok))
                    else:
                        out.stop_reason = reason
                        out.decode_duration = time.perf_counter() - t_decode
                        held.discard(s)
                        stepper.end_sequence(s)
                if not going:
                    if ahead is not None:
                        collect(ahead)      # nobody is left to use it
                    break
                slots_now = [s for _, s, _ in going]
                if ahead is not None and len(going) < len(live):
                    # the step that is already running was fed with the tokens judged above:
                    # the rows of the sequences that go on are the ones they need
                    row = {s: t for (_, s, _), t in zip(live, collect(ahead))}
                    live = [(i, s, int(row[s])) for i, s, _ in going]
                    ahead = None
                    continue
                ticket = ahead if ahead is not None else issue(
                    slots_now, [t for _, _, t in going], config.sampling)
                ahead = None
                if ahead_ok and stepper.can_feed_back(slots_now, config.sampling) and all(
                        stepper.length(s) < max_seq_len for s in slots_now) and any(
                        limit < 0 or len(results[i].token_ids) + 1 < limit for i, _, _ in going):
                    # the step after this one, for as long as any sequence could use its token
                    ahead = issue(slots_now, None, config.sampling)
                live = [(i, s, int(t)) for (i, s, _), t in zip(going, collect(ticket))]
        except BaseException:
            for s in held:      # give back what the failed batch still holds
                stepper.end_sequence(s)
            raise
    return results  # type: ignore[return-value]
