"""The generation loop's decisions, with a scripted stepper instead of a model
(no device needed).  The cases follow the reference's own loop tests
(src/engine/generate.rs:1594-2111): max tokens, stop token not emitted,
context stop keeps the last token, cancellation keeps the token, empty and
too-long prompts, and what the reference has no counterpart for: batches,
early finishers and slots that are used again."""

import pytest

from strata_inference_b200.engine.generate import (CANCELLED, CONTEXT_LENGTH, MAX_TOKENS,
                                                   STOP_TOKEN, GenerationConfig, GenerationError,
                                                   generate, plan_batch)
from strata_inference_b200.sampling.sampler import SamplingConfig


class ScriptedStepper:
    """The next token of a sequence is ``script(prompt, n_fed)``; slots and
    lengths are tracked as a cache would."""

    def __init__(self, script, max_seq_len=64, capacity_tokens=1 << 20, slots=8, page_tokens=64,
                 stops=()):
        self.script = script
        self.max_seq_len = max_seq_len
        self.page_tokens = page_tokens
        self.default_stop_tokens = tuple(stops)
        self._capacity = capacity_tokens
        self._free = list(range(slots - 1, -1, -1))
        self.live = {}            # slot -> [prompt, fed tokens]
        self.seeds = {}
        self.log = []             # ("prefill", slots) / ("decode", slots)
        self.acquired = []

    @property
    def capacity_tokens(self):
        return self._capacity

    @property
    def free_slots(self):
        return len(self._free)

    def new_sequence(self):
        s = self._free.pop()
        assert s not in self.live
        self.live[s] = None
        self.acquired.append(s)
        return s

    def end_sequence(self, slot):
        assert slot in self.live, "freed twice"
        del self.live[slot]
        self._free.append(slot)

    def length(self, slot):
        prompt, fed = self.live[slot]
        return len(prompt) + len(fed)

    def seed(self, slot, seed):
        self.seeds[slot] = seed

    def prefill(self, slots, prompts, sampling):
        self.log.append(("prefill", list(slots)))
        for s, p in zip(slots, prompts):
            self.live[s] = [list(p), []]
        return [self.script(self.live[s][0], 0) for s in slots]

    def decode(self, slots, tokens, sampling):
        self.log.append(("decode", list(slots)))
        out = []
        for s, t in zip(slots, tokens):
            assert self.length(s) < self.max_seq_len, "fed beyond the context"
            self.live[s][1].append(t)
            out.append(self.script(self.live[s][0], len(self.live[s][1])))
        return out


def counting(prompt, n_fed):
    return 100 + n_fed


def test_max_tokens_and_zero():
    st = ScriptedStepper(counting)
    out = generate(st, [[1, 2, 3]], GenerationConfig(max_tokens=4))[0]
    assert out.token_ids == [100, 101, 102, 103] and out.stop_reason == MAX_TOKENS
    assert out.prompt_tokens == 3 and not st.live
    out = generate(st, [[1, 2, 3]], GenerationConfig(max_tokens=0))[0]
    assert out.token_ids == [] and out.stop_reason == MAX_TOKENS


def test_stop_token_is_not_emitted():
    st = ScriptedStepper(counting, stops=(103,))
    seen = []
    out = generate(st, [[5]], GenerationConfig(max_tokens=50), lambda i, t: seen.append(t) or True)[0]
    assert out.token_ids == [100, 101, 102] and out.stop_reason == STOP_TOKEN and seen == out.token_ids
    out = generate(st, [[5]], GenerationConfig(max_tokens=50, stop_tokens=[101]))[0]
    assert out.token_ids == [100] and out.stop_reason == STOP_TOKEN
    out = generate(st, [[5]], GenerationConfig(max_tokens=50, stop_tokens=[100]))[0]
    assert out.token_ids == [] and out.stop_reason == STOP_TOKEN


def test_context_end_keeps_the_last_token_and_never_feeds_it():
    st = ScriptedStepper(counting, max_seq_len=5)
    out = generate(st, [[1, 2]], GenerationConfig(max_tokens=-1))[0]
    # prompt 2 + fed 3 = 5 positions; the fourth token is produced but not fed
    assert out.token_ids == [100, 101, 102, 103] and out.stop_reason == CONTEXT_LENGTH


def test_cancel_keeps_the_token():
    st = ScriptedStepper(counting)
    out = generate(st, [[1]], GenerationConfig(max_tokens=10), lambda i, t: t != 102)[0]
    assert out.token_ids == [100, 101, 102] and out.stop_reason == CANCELLED and not st.live


def test_prompt_errors():
    st = ScriptedStepper(counting, max_seq_len=4)
    with pytest.raises(GenerationError, match="empty"):
        generate(st, [[1], []], GenerationConfig())
    with pytest.raises(GenerationError, match="exceeds max_seq_len"):
        generate(st, [[1, 2, 3, 4]], GenerationConfig())
    assert generate(st, [], GenerationConfig()) == []
    assert not st.acquired


def test_unequal_batch_early_finishers_leave_and_free_their_slots():
    stops = {3: 102, 1: 100}          # by prompt length: when each request stops

    def script(prompt, n_fed):
        tok = 100 + n_fed
        return 999 if stops.get(len(prompt)) == tok else tok
    st = ScriptedStepper(script, stops=(999,))
    outs = generate(st, [[1, 1, 1], [2], [3, 3]], GenerationConfig(max_tokens=5))
    assert [o.token_ids for o in outs] == [[100, 101], [], [100, 101, 102, 103, 104]]
    assert [o.stop_reason for o in outs] == [STOP_TOKEN, STOP_TOKEN, MAX_TOKENS]
    kinds = [(k, len(s)) for k, s in st.log]
    assert kinds == [("prefill", 3), ("decode", 2), ("decode", 2), ("decode", 1), ("decode", 1)]
    assert not st.live and st.free_slots == 8


def test_more_requests_than_fit_run_as_batches_one_after_another():
    st = ScriptedStepper(counting, slots=2)
    outs = generate(st, [[1], [2, 2], [3], [4], [5]], GenerationConfig(max_tokens=2))
    assert all(o.token_ids == [100, 101] for o in outs)
    assert [k for k, _ in st.log if k == "prefill"] == ["prefill"] * 3
    assert [len(s) for k, s in st.log if k == "prefill"] == [2, 2, 1]
    assert len(set(st.acquired)) == 2 and len(st.acquired) == 5     # slots used again


def test_plan_batch_counts_whole_pages_to_each_request_s_end():
    assert plan_batch([10, 10, 10], 20, 4096, 64, 128, 8) == 2       # 64 positions each
    assert plan_batch([100, 10], 100, 4096, 64, 256, 8) == 1          # 256, then no room
    assert plan_batch([10, 10], -1, 128, 64, 256, 8) == 2             # to the context end
    assert plan_batch([10, 10, 10], 5, 4096, 64, 1 << 20, 2) == 2     # slots
    with pytest.raises(GenerationError, match="does not fit"):
        plan_batch([1000], 10, 4096, 64, 512, 8)


def test_every_request_gets_its_seed():
    st = ScriptedStepper(counting)
    generate(st, [[1], [2]], GenerationConfig(max_tokens=1, sampling=SamplingConfig(0.7, seed=9)))
    assert sorted(st.seeds.values()) == [9, 9]
    st = ScriptedStepper(counting)
    generate(st, [[1], [2]], GenerationConfig(max_tokens=1), seeds=[3, 4])
    assert sorted(st.seeds.values()) == [3, 4]
    st = ScriptedStepper(counting)
    generate(st, [[1]], GenerationConfig(max_tokens=1))
    assert list(st.seeds.values()) == [42]                          # the reference's default


def test_a_failing_step_gives_the_slots_back():
    def boom(prompt, n_fed):
        if n_fed == 2:
            raise RuntimeError("device fault")
        return 100 + n_fed
    st = ScriptedStepper(boom)
    with pytest.raises(RuntimeError, match="device fault"):
        generate(st, [[1], [2, 2]], GenerationConfig(max_tokens=10))
    assert not st.live and st.free_slots == 8


def test_the_fast_layout_of_single_token_steps_is_the_general_one():
    import numpy as np
    from strata_inference_b200.parts.base import StepContext
    slots, lengths, tokens = [5, 0, 9, 2], [17, 300, 0, 64], [11, 7, 400, 3]
    out = np.full((8, 4), -7, dtype=np.int32)
    StepContext.pack_single_tokens(out, slots, lengths, tokens)
    general = StepContext.pack([(s, n, 1) for s, n in zip(slots, lengths)], tokens, range(4))
    assert general.dtype == np.int32 and general.tolist() == out.reshape(-1).tolist()
    assert StepContext.packed_size(4, 4, 4) == out.size


class LookAheadStepper(ScriptedStepper):
    """A scripted stepper that can launch a step and hand its tokens out later, and feed a
    step with what the step before sampled: what the loop needs to stay one step ahead."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.last = None          # (slots, tokens) of the latest launched step
        self.open = 0
        self.fed_back = 0

    def decode_issue(self, slots, tokens, sampling):
        if tokens is None:
            assert self.can_feed_back(slots, sampling), "nothing to feed back"
            tokens = self.last[1]
            self.fed_back += 1
        out = super().decode(slots, tokens, sampling)
        self.last = (list(slots), out)
        self.open += 1
        assert self.open <= 2, "more than one step ahead"
        return out

    def decode_collect(self, ticket):
        self.open -= 1
        return ticket

    def can_feed_back(self, slots, sampling):
        # (a slot that has ended since cannot be in `slots`: the loop asks for live ones)
        return self.last is not None and self.last[0] == list(slots)

    def prefill(self, slots, prompts, sampling):
        self.last = None
        return super().prefill(slots, prompts, sampling)


def _ragged(prompt, n_fed):
    """Tokens that depend on the prompt and the place; token 7 ends a sequence."""
    v = (prompt[0] * 31 + n_fed * 17 + len(prompt)) % 23
    return 7 if v == 0 and n_fed > 1 else 100 + v


@pytest.mark.parametrize("limit", [0, 1, 2, 5, 40, -1])
def test_looking_one_step_ahead_changes_no_decision(limit):
    prompts = [[k + 1] * (3 + 5 * k % 11) for k in range(7)]
    conf = GenerationConfig(max_tokens=limit, stop_tokens=[7])
    cancel_at = {2: 4, 5: 1}      # request -> emitted tokens after which it cancels

    def run(stepper, look_ahead):
        seen = {}

        def cb(i, t):
            seen[i] = seen.get(i, 0) + 1
            return seen[i] != cancel_at.get(i)
        outs = generate(stepper, prompts, GenerationConfig(limit, [7], conf.sampling, look_ahead), cb)
        assert not stepper.live, "a slot was not given back"
        return [(o.token_ids, o.stop_reason) for o in outs]

    plain = run(ScriptedStepper(_ragged, max_seq_len=30, slots=3), False)
    ahead = LookAheadStepper(_ragged, max_seq_len=30, slots=3)
    assert run(ahead, True) == plain
    assert ahead.open == 0
    if limit < 0 or limit > 2:
        assert ahead.fed_back > 0          # it did look ahead
    off = LookAheadStepper(_ragged, max_seq_len=30, slots=3)
    assert run(off, False) == plain and off.fed_back == 0
    reasons = {r for _, r in plain}
    if limit < 0:
        assert {STOP_TOKEN, CANCELLED, CONTEXT_LENGTH} <= reasons
