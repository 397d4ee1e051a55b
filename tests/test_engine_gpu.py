"""The engine against the plain implementation, in 32-bit and in bfloat16:
each request alone and whole; with its last 32 tokens one by one; in batches
of unequal lengths whose shorter requests end earlier, one batch after
another so that slots are used again; long decoding; the first tokens."""

import pytest
import torch

from helpers import (CONFIGS, SHARPEN, assert_logits_close, make_model_dir, plain_logits,
                     random_prompts)

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
# (config, page size): the small page sizes make the window's ring wrap
CASES = [("A", 64), ("A", 4), ("B", 64), ("B", 8), ("C", 16)]


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        for dtype, sharpen in SHARPEN.items():
            out[name, dtype] = make_model_dir(str(tmp_path_factory.mktemp(f"tiny_{name}_{dtype}")),
                                              cfg, seed=10 + i, sharpen=sharpen)
    return out


def _engine(model_dirs, name, dtype, page_tokens, max_tokens=1024):
    from strata_inference_b200 import Engine
    return Engine.from_dir(model_dirs[name, dtype], dtype=dtype, max_tokens=max_tokens,
                           page_tokens=page_tokens)


def _lengths(cfg):
    top = cfg["max_position_embeddings"]
    return [top - 3, 40, top // 2 + 5]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", CASES)
def test_whole_prompt_each_request_alone(model_dirs, name, page, dtype):
    cfg = CONFIGS[name]
    eng = _engine(model_dirs, name, dtype, page)
    for r, toks in enumerate(random_prompts(cfg, _lengths(cfg), seed=1)):
        ref = plain_logits(toks, model_dirs[name, dtype], cfg)
        slot = eng.new_sequence()
        got = eng.step([(slot, toks)], want=[list(range(len(toks)))])
        eng.end_sequence(slot)
        assert_logits_close(got, ref, dtype, f"{name} request {r} whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", CASES)
def test_last_32_tokens_one_by_one(model_dirs, name, page, dtype):
    cfg = CONFIGS[name]
    eng = _engine(model_dirs, name, dtype, page)
    for r, toks in enumerate(random_prompts(cfg, _lengths(cfg), seed=2)):
        ref = plain_logits(toks, model_dirs[name, dtype], cfg)
        cut = len(toks) - 32
        slot = eng.new_sequence()
        got = [eng.step([(slot, toks[:cut])], want=[[cut - 1]])]
        for t in toks[cut:]:
            got.append(eng.step([(slot, [t])]))
        eng.end_sequence(slot)
        got = torch.cat(got, dim=0)
        assert_logits_close(got, ref[cut - 1:], dtype, f"{name} request {r} last 32 one by one")


def _run_batch(eng, requests, prompt_lens, refs, dtype, tag):
    """Prompts of unequal lengths in one step, then one given token each per
    step; a request leaves (and frees its slot) when its tokens are used up."""
    slots = [eng.new_sequence() for _ in requests]
    entries = [(s, toks[:p]) for s, toks, p in zip(slots, requests, prompt_lens)]
    want = [[0, p - 1] if p > 1 else [0] for p in prompt_lens]
    got = eng.step(entries, want)
    ref = torch.cat([refs[i][w] for i, w in enumerate(want)], dim=0)
    assert_logits_close(got, ref, dtype, f"{tag} prompts")
    pos = list(prompt_lens)
    live = list(range(len(requests)))
    step = 0
    while live:
        still = [i for i in live if pos[i] < len(requests[i])]
        for i in live:
            if i not in still:
                eng.end_sequence(slots[i])
        live = still
        if not live:
            break
        got = eng.step([(slots[i], [requests[i][pos[i]]]) for i in live])
        ref = torch.stack([refs[i][pos[i]] for i in live], dim=0)
        assert_logits_close(got, ref, dtype, f"{tag} decode step {step} (requests {live})")
        for i in live:
            pos[i] += 1
        step += 1
    return slots


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", CASES)
def test_unequal_batches_one_after_another(model_dirs, name, page, dtype):
    cfg = CONFIGS[name]
    top = cfg["max_position_embeddings"]
    eng = _engine(model_dirs, name, dtype, page, max_tokens=4 * ((top + 63) // 64) * 64)
    total = [top - 1, 30, 45, 37, top - 10, 12, 50]
    prompt = [20, 3, 33, 1, top - 30, 11, 9]
    reqs = random_prompts(cfg, total, seed=3)
    refs = [plain_logits(t, model_dirs[name, dtype], cfg) for t in reqs]
    first = _run_batch(eng, reqs[:4], prompt[:4], refs[:4], dtype, f"{name} batch 1")
    assert eng.cache.pages_in_use() == 0
    second = _run_batch(eng, reqs[4:], prompt[4:], refs[4:], dtype, f"{name} batch 2")
    assert set(second) & set(first), "the second batch should reuse slots of the first"
    assert eng.cache.pages_in_use() == 0 and eng.cache.n_free_slots == eng.cache.max_slots


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model_dirs, dtype):
    """A 2-token prompt, then every further token one by one up to the context's end."""
    name, cfg = "C", CONFIGS["C"]
    eng = _engine(model_dirs, name, dtype, 16)
    toks = random_prompts(cfg, [cfg["max_position_embeddings"]], seed=4)[0]
    ref = plain_logits(toks, model_dirs[name, dtype], cfg)
    slot = eng.new_sequence()
    got = [eng.step([(slot, toks[:2])], want=[[0, 1]])]
    for t in toks[2:]:
        got.append(eng.step([(slot, [t])]))
    assert_logits_close(torch.cat(got, dim=0), ref, dtype, "C long decoding")
    with pytest.raises(Exception):
        eng.step([(slot, [1])])   # the context is full
    eng.end_sequence(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens(model_dirs, name, dtype):
    """Position 0 alone, then positions 1, 2, 3 one by one, and a one-token
    prompt beside longer ones."""
    cfg = CONFIGS[name]
    eng = _engine(model_dirs, name, dtype, 64)
    toks = random_prompts(cfg, [4], seed=5)[0]
    ref = plain_logits(toks, model_dirs[name, dtype], cfg)
    slot = eng.new_sequence()
    got = torch.cat([eng.step([(slot, [t])]) for t in toks], dim=0)
    eng.end_sequence(slot)
    assert_logits_close(got, ref, dtype, f"{name} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8), ("C", 16)])
def test_prompts_continued_in_pieces(model_dirs, name, page, dtype):
    """Two requests fed in pieces of unequal sizes (several new positions of a sequence in one
    step, below and above the number of rows the weight-streaming kernels take): the logits
    of every position are those of the whole prompt."""
    cfg = CONFIGS[name]
    eng = _engine(model_dirs, name, dtype, page)
    top = cfg["max_position_embeddings"]
    a, b = random_prompts(cfg, [top - 2, top // 2], seed=6)
    ref_a = plain_logits(a, model_dirs[name, dtype], cfg)
    ref_b = plain_logits(b, model_dirs[name, dtype], cfg)
    # a sequence may add at most (ring - window + 1) positions a step once it has begun
    most = eng.cache.max_step_tokens()
    sa, sb = eng.new_sequence(), eng.new_sequence()
    pa = pb = 0
    pieces = [(5, 3), (1, 2), (7, 1), (3, 6), (2, 2), (9, 4), (20, 1), (4, 3)]
    k = 0
    got_a, got_b = [], []
    while pa < len(a) or pb < len(b):
        na, nb = pieces[k % len(pieces)]
        k += 1
        if pa > 0:
            na = min(na, most)
        if pb > 0:
            nb = min(nb, most)
        na, nb = min(na, len(a) - pa), min(nb, len(b) - pb)
        entries, want = [], []
        if na:
            entries.append((sa, a[pa:pa + na]))
            want.append(list(range(na)))
        if nb:
            entries.append((sb, b[pb:pb + nb]))
            want.append(list(range(nb)))
        out = eng.step(entries, want=want)          # both begin in the first step, then both go on
        if na:
            got_a.append(out[:na])
        if nb:
            got_b.append(out[na:na + nb])
        pa, pb = pa + na, pb + nb
    eng.end_sequence(sa)
    eng.end_sequence(sb)
    assert_logits_close(torch.cat(got_a), ref_a, dtype, f"{name} request a in pieces")
    assert_logits_close(torch.cat(got_b), ref_b, dtype, f"{name} request b in pieces")
    assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_key_and_window_edge(tmp_path, dtype):
    """One early key made to stand out: a global layer must find it among all
    keys, a sliding layer must lose it exactly when it leaves the window."""
    from strata_inference_b200 import Engine
    cfg = dict(CONFIGS["A"])
    cfg["max_position_embeddings"] = 256
    cfg["sliding_window"] = 24
    d = make_model_dir(str(tmp_path / "m"), cfg, seed=21, sharpen=1.5 * SHARPEN[dtype])
    toks = random_prompts(cfg, [200], seed=6)[0]
    toks[5] = 77                      # a token that appears once, early
    toks = [t if (t != 77 or i == 5) else 78 for i, t in enumerate(toks)]
    ref = plain_logits(toks, d, cfg)
    eng = Engine.from_dir(d, dtype=dtype, max_tokens=512, page_tokens=8)
    slot = eng.new_sequence()
    got = [eng.step([(slot, toks[:20])], want=[list(range(20))])]
    for t in toks[20:]:
        got.append(eng.step([(slot, [t])]))
    eng.end_sequence(slot)
    assert_logits_close(torch.cat(got, dim=0), ref, dtype, "far key / window edge")


def test_padding_free_batch_is_independent_of_neighbours(model_dirs):
    """The same request gives the same logits alone and beside others (32-bit)."""
    name, cfg = "B", CONFIGS["B"]
    eng = _engine(model_dirs, name, "float32", 8)
    reqs = random_prompts(cfg, [17, 5, 29], seed=7)
    alone = []
    for t in reqs:
        s = eng.new_sequence()
        alone.append(eng.step([(s, t)]))
        eng.end_sequence(s)
    slots = [eng.new_sequence() for _ in reqs]
    together = eng.step(list(zip(slots, reqs)))
    for s in slots:
        eng.end_sequence(s)
    scale = torch.cat(alone).abs().max().item()
    assert (together - torch.cat(alone)).abs().max().item() <= 1e-5 * scale


def test_step_errors(model_dirs):
    from strata_inference_b200.cache.paged import CacheError, CacheFull
    name, cfg = "A", CONFIGS["A"]
    eng = _engine(model_dirs, name, "float32", 64, max_tokens=128)
    s = eng.new_sequence()
    with pytest.raises(ValueError, match="exceeds vocab_size"):
        eng.step([(s, [cfg["vocab_size"]])])
    with pytest.raises(ValueError):
        eng.step([(s, [])])
    with pytest.raises(ValueError, match="twice"):
        eng.step([(s, [1]), (s, [2])])
    eng.step([(s, [1, 2, 3])])
    s2 = eng.new_sequence()
    with pytest.raises(CacheFull):
        eng.step([(s2, list(range(100)))])      # 2 pages wanted, 1 free
    assert eng.length(s2) == 0
    eng.end_sequence(s)
    eng.end_sequence(s2)
    with pytest.raises(CacheError):
        eng.end_sequence(s2)
    with pytest.raises(CacheError):
        eng.step([(s2, [1])])


# Sizes at the edges of what the fast kernels take: a width that is no multiple of 8 (no
# 16-byte rows), an intermediate size that is no multiple of 8 (gate and up rows cannot be
# interleaved), three heads to a kv head, head sizes 80 and 112, an odd vocabulary.
ODD = {
    "narrow rows": dict(hidden_size=100, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                        intermediate_size=100, vocab_size=257),
    "three to a group": dict(hidden_size=72, num_attention_heads=6, num_key_value_heads=2,
                             head_dim=80, intermediate_size=88, vocab_size=301),
    "seven heads": dict(hidden_size=88, num_attention_heads=7, num_key_value_heads=7, head_dim=112,
                        intermediate_size=136, vocab_size=130),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(ODD))
def test_sizes_the_fast_kernels_refuse_take_the_general_ones(tmp_path, which, dtype):
    from strata_inference_b200 import Engine
    cfg = dict(CONFIGS["A"], **ODD[which], max_position_embeddings=96, sliding_window=20,
               query_pre_attn_scalar=ODD[which]["head_dim"])
    d = make_model_dir(str(tmp_path / "odd"), cfg, seed=31, sharpen=SHARPEN[dtype])
    eng = Engine.from_dir(d, dtype=dtype, max_tokens=512, page_tokens=16)
    a, b = random_prompts(cfg, [70, 33], seed=7)
    ref_a, ref_b = plain_logits(a, d, cfg), plain_logits(b, d, cfg)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    got = eng.step([(sa, a[:40]), (sb, b[:9])], want=[list(range(40)), list(range(9))])
    assert_logits_close(got, torch.cat([ref_a[:40], ref_b[:9]]), dtype, f"{which}: prompts")
    for t in range(24):
        got = eng.step([(sa, [a[40 + t]]), (sb, [b[9 + t]])])
        assert_logits_close(got, torch.stack([ref_a[40 + t], ref_b[9 + t]]), dtype,
                            f"{which}: step {t}")
    eng.end_sequence(sb)
    got = eng.step([(sa, a[64:])], want=[list(range(6))])
    assert_logits_close(got, ref_a[64:], dtype, f"{which}: tail")
    eng.end_sequence(sa)


def test_steps_issued_without_waiting_and_a_scratch_buffer_that_grows(model_dirs):
    """Single-token steps issued back to back, their results read only at the end: every step
    sees its own positions (the metadata's staging buffers are not rewritten before they were
    copied).  And the scratch buffer that a captured step writes into is not given back when a
    later step needs a larger one: memory allocated afterwards stays untouched by replays."""
    name, dtype = "A", "bfloat16"
    cfg = CONFIGS[name]
    eng = _engine(model_dirs, name, dtype, 16)
    toks = random_prompts(cfg, [100], seed=8)[0]
    ref = plain_logits(toks, model_dirs[name, dtype], cfg)
    slot = eng.new_sequence()
    eng.step([(slot, toks[:60])])
    for t in toks[60:64]:                       # eager step, capture, two replays
        eng.decode_step([slot], [t])
    small = eng.rt.scratch(1)
    eng.rt.scratch(4 * small.numel())           # a later step needs more
    assert eng.rt.scratch(1).data_ptr() != small.data_ptr()
    del small
    victims = [torch.zeros(1 << 18, dtype=torch.uint8, device=eng.device) for _ in range(8)]
    got = []
    for t in toks[64:96]:
        eng.decode_step([slot], [t])
        got.append(eng.last_logits.clone())     # no wait for the device in this loop
    eng.end_sequence(slot)
    assert all(int(v.sum()) == 0 for v in victims), "a replay wrote into memory that is not its own"
    assert_logits_close(torch.cat(got), ref[64:96], dtype, "steps issued without waiting")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_batch_of_twenty(model_dirs, name, dtype):
    """More sequences than the weight-streaming kernels take rows: the single-token steps of
    20 sequences go through the library products, the rotation kernel and the cache
    attention with 20 rows; through `step` and through the captured `decode_step`."""
    cfg = CONFIGS[name]
    eng = _engine(model_dirs, name, dtype, 16, max_tokens=4096)
    lens = [5 + (7 * i) % 26 for i in range(20)]
    reqs = random_prompts(cfg, [n + 8 for n in lens], seed=9)
    refs = [plain_logits(t, model_dirs[name, dtype], cfg) for t in reqs]
    slots = [eng.new_sequence() for _ in reqs]
    got = eng.step([(s, r[:n]) for s, r, n in zip(slots, reqs, lens)])
    assert_logits_close(got, torch.stack([f[n - 1] for f, n in zip(refs, lens)]), dtype,
                        f"{name}: 20 prompts")
    for k in range(8):
        toks = [r[n + k] for r, n in zip(reqs, lens)]
        if k < 4:
            got = eng.step([(s, [t]) for s, t in zip(slots, toks)])
        else:
            eng.decode_step(slots, toks)
            got = eng.last_logits
        assert_logits_close(got, torch.stack([f[n + k] for f, n in zip(refs, lens)]), dtype,
                            f"{name}: 20 sequences, step {k}")
    for s in slots:
        eng.end_sequence(s)
    assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page,room", [("A", 4, 40), ("B", 8, 12), ("C", 16, 100)])
def test_prompts_continued_in_pieces_larger_than_a_page(model_dirs, name, page, room, dtype):
    """A cache built with room for long continuing steps (`max_continuation`): prompts are
    fed in pieces much larger than a page and than the window, across the ring's end, and a
    piece beyond the room is refused with the figure in the message."""
    from strata_inference_b200 import Engine
    from strata_inference_b200.engine.engine import StepError
    cfg = CONFIGS[name]
    eng = Engine.from_dir(model_dirs[name, dtype], dtype=dtype, max_tokens=1024, page_tokens=page,
                          max_continuation=room)
    ring = [g for g in eng.cache.groups if g.need.window][0]
    assert ring.ring_tokens > 0, "the window's group must be a ring for this test to mean anything"
    most = eng.cache.max_step_tokens()
    assert room <= most < room + page
    top = cfg["max_position_embeddings"]
    a, b = random_prompts(cfg, [top - 1, top - 7], seed=16)
    ref_a = plain_logits(a, model_dirs[name, dtype], cfg)
    ref_b = plain_logits(b, model_dirs[name, dtype], cfg)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    first = (3, 11)
    out = eng.step([(sa, a[:first[0]]), (sb, b[:first[1]])],
                   want=[list(range(first[0])), list(range(first[1]))])
    got_a, got_b = [out[:first[0]]], [out[first[0]:]]
    pa, pb = first
    refused = False
    while pa < len(a) or pb < len(b):
        if not refused and pa + most + 1 > ring.ring_tokens and pa + most + 1 <= len(a):
            # one position more than the room, where it would wrap around the ring
            with pytest.raises(StepError, match=f"at most {most} "):
                eng.step([(sa, a[pa:pa + most + 1])])
            assert eng.length(sa) == pa
            refused = True
        na, nb = min(most, len(a) - pa), min(max(1, most - 5), len(b) - pb)
        entries = [(s, t[p:p + n]) for s, t, p, n in ((sa, a, pa, na), (sb, b, pb, nb)) if n]
        out = eng.step(entries, want=[list(range(len(t))) for _, t in entries])
        if na:
            got_a.append(out[:na])
        if nb:
            got_b.append(out[na:na + nb])
        pa, pb = pa + na, pb + nb
    eng.end_sequence(sa)
    eng.end_sequence(sb)
    assert refused
    assert_logits_close(torch.cat(got_a), ref_a, dtype, f"{name} request a in long pieces")
    assert_logits_close(torch.cat(got_b), ref_b, dtype, f"{name} request b in long pieces")
    assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8), ("C", 16)])
def test_a_new_prompt_beside_sequences_that_go_on(model_dirs, name, page, dtype):
    """A mixed step: one sequence starts (its whole prompt, from position 0, longer than the
    window) in the step in which two others go on by one token and by several.  The new
    sequence's rows then attend over the cache like any other continuing rows."""
    cfg = CONFIGS[name]
    eng = _engine(model_dirs, name, dtype, page)
    a, b, c = random_prompts(cfg, [50, 44, 58], seed=17)
    refs = [plain_logits(t, model_dirs[name, dtype], cfg) for t in (a, b, c)]
    sa, sb = eng.new_sequence(), eng.new_sequence()
    eng.step([(sa, a[:30]), (sb, b[:21])])
    most = eng.cache.max_step_tokens()
    few = min(3, most)
    sc = eng.new_sequence()
    n_c = min(40, eng.cache.max_step_tokens(0))       # a prompt may fill the ring once
    got = eng.step([(sa, a[30:31]), (sc, c[:n_c]), (sb, b[21:21 + few])],
                   want=[[0], list(range(n_c)), list(range(few))])
    ref = torch.cat([refs[0][30:31], refs[2][:n_c], refs[1][21:21 + few]])
    assert_logits_close(got, ref, dtype, f"{name} mixed step")
    # all three go on by one token: the new sequence's cache is as good as the others'
    pa, pb, pc = 31, 21 + few, n_c
    for k in range(6):
        got = eng.step([(sa, [a[pa + k]]), (sb, [b[pb + k]]), (sc, [c[pc + k]])])
        ref = torch.stack([refs[0][pa + k], refs[1][pb + k], refs[2][pc + k]])
        assert_logits_close(got, ref, dtype, f"{name} after the mixed step, token {k}")
    for s in (sa, sb, sc):
        eng.end_sequence(s)
    assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_failed_step_leaves_the_cache_as_it_was(model_dirs, dtype):
    """A step whose forward pass raises gives back the pages it reserved and advances
    nothing; the same slot then runs the same tokens as a fresh engine would."""
    name, cfg = "B", CONFIGS["B"]
    eng = _engine(model_dirs, name, dtype, 8)
    toks = random_prompts(cfg, [40], seed=18)[0]
    ref = plain_logits(toks, model_dirs[name, dtype], cfg)
    s = eng.new_sequence()
    eng.step([(s, toks[:10])])
    held = eng.cache.pages_in_use()
    first_block = eng.model.blocks[0]
    real = first_block.forward

    def broken(*a, **kw):
        raise RuntimeError("made to fail")
    first_block.forward = broken
    with pytest.raises(RuntimeError, match="made to fail"):
        eng.step([(s, toks[10:19])])
    with pytest.raises(RuntimeError, match="made to fail"):
        eng.decode_step([s], [toks[10]])
    first_block.forward = real
    assert eng.cache.pages_in_use() == held and eng.length(s) == 10
    got = [eng.step([(s, toks[10:14])], want=[list(range(4))])]
    for t in toks[14:]:
        got.append(eng.step([(s, [t])]))
    eng.end_sequence(s)
    assert_logits_close(torch.cat(got), ref[10:], dtype, "after a failed step")
    assert eng.cache.pages_in_use() == 0


def test_a_kernel_that_gave_up_is_reported_and_the_slots_come_back(model_dirs):
    """The bounded waits of the tcgen05 kernels leave a code in a device word when they run
    out.  Here the word is set from the host (nothing is made to stall): the generation
    loop learns of it where it reads the sampled tokens, raises, and frees its slots."""
    from strata_inference_b200 import GenerationConfig, GenerationEngine
    from strata_inference_b200.kernels import native
    name = "A"
    gen = GenerationEngine.from_dir(model_dirs[name, "bfloat16"], dtype="bfloat16", max_tokens=512)
    prompts = random_prompts(CONFIGS[name], [9, 4], seed=19)
    want = [o.token_ids for o in gen.generate(prompts, GenerationConfig(max_tokens=6))]
    native.set_kernel_error(1, 2)              # "attention_prefill_tc: a load never arrived"
    with pytest.raises(native.KernelError, match="attention_prefill_tc.*code 2"):
        gen.generate(prompts, GenerationConfig(max_tokens=6))
    cache = gen.engine.cache
    assert cache.n_free_slots == cache.max_slots and cache.pages_in_use() == 0
    # the word was cleared with the report: the engine works again
    assert [o.token_ids for o in gen.generate(prompts, GenerationConfig(max_tokens=6))] == want
    native.set_kernel_error(0, 3)              # during decoding: found at the next token read
    seen = []

    def on_token(i, t):
        seen.append(t)
        if len(seen) == 4:
            native.set_kernel_error(0, 3)
        return True
    native.set_kernel_error(0, 0)
    with pytest.raises(native.KernelError, match="gemm_tcgen05.*code 3"):
        gen.generate(prompts, GenerationConfig(max_tokens=6), on_token)
    assert cache.n_free_slots == cache.max_slots and cache.pages_in_use() == 0


def test_captured_steps_are_kept_for_a_few_batch_sizes_only(model_dirs):
    name, cfg = "A", CONFIGS["A"]
    eng = _engine(model_dirs, name, "bfloat16", 16, max_tokens=4096)
    eng.max_graphs = 3
    slots = [eng.new_sequence() for _ in range(6)]
    eng.step([(s, [3, 4, 5]) for s in slots])
    for n in (6, 5, 4, 3, 2, 6):
        for _ in range(3):
            eng.decode_step(slots[:n], [7] * n)
    assert len(eng._graphs) == 3 and [k[0] for k in eng._graphs] == [3, 2, 6]


@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8), ("C", 16)])
def test_steps_of_few_rows_as_one_chain_kernel(model_dirs, name, page):
    """The optional chain kernel (everything between two attention kernels of a step of at
    most 16 rows as one launch, deferred steps collected by the runtime): prompts of few
    tokens, single tokens of unequal batches, captured steps; bfloat16."""
    from strata_inference_b200 import Engine
    dtype = "bfloat16"
    cfg = CONFIGS[name]
    eng = Engine.from_dir(model_dirs[name, dtype], dtype=dtype, max_tokens=1024, page_tokens=page)
    eng.rt.chain_steps = True
    reqs = random_prompts(cfg, [40, 28, 35], seed=23)
    refs = [plain_logits(t, model_dirs[name, dtype], cfg) for t in reqs]
    slots = [eng.new_sequence() for _ in reqs]
    first = [5, 3, 7]                                   # 15 rows: the prompts go through the chain too
    got = eng.step([(s, r[:n]) for s, r, n in zip(slots, reqs, first)],
                   want=[list(range(n)) for n in first])
    assert_logits_close(got, torch.cat([f[:n] for f, n in zip(refs, first)]), dtype, f"{name} prompts")
    pos = list(first)
    before = eng.rt.chain_sync().clone()
    for k in range(20):
        toks = [r[p] for r, p in zip(reqs, pos)]
        if k < 10:
            got = eng.step([(s, [t]) for s, t in zip(slots, toks)])
        else:
            eng.decode_step(slots, toks)                # captured from the second one on
            got = eng.last_logits
        assert_logits_close(got, torch.stack([f[p] for f, p in zip(refs, pos)]), dtype,
                            f"{name} chained step {k}")
        pos = [p + 1 for p in pos]
    assert eng.rt.chain_sync().tolist() == before.tolist() == [0, 0]
    for s in slots:
        eng.end_sequence(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8), ("C", 16)])
def test_short_prompt_steps_replayed_from_a_recording(model_dirs, name, page, dtype):
    """Steps of two prompts with 17 to 64 rows in all share one recorded step (rows are
    filled up to 64 with a sequence that holds no slot): launched one by one twice, then
    replayed.  Every step brings other lengths, slots and wanted places; the logits at the
    wanted places and those of two more tokens decoded from what the step left in the
    cache equal the plain implementation's, and no page is lost."""
    cfg = CONFIGS[name]
    eng = _engine(model_dirs, name, dtype, page)
    lens = [(20, 30), (5, 12), (40, 24), (1, 60), (33, 9), (16, 16)]
    held = []
    for i, (a, b) in enumerate(lens):
        reqs = random_prompts(cfg, [a + 2, b + 2], seed=70 + i)
        refs = [plain_logits(t, model_dirs[name, dtype], cfg) for t in reqs]
        if i == 3:      # other slots than before: the ones held so far stay taken
            held = [eng.new_sequence() for _ in range(2)]
        slots = [eng.new_sequence(), eng.new_sequence()]
        want = [[a // 2, a - 1], [b - 1, 0]]
        got = eng.step([(slots[0], reqs[0][:a]), (slots[1], reqs[1][:b])], want)
        ref = torch.stack([refs[0][a // 2], refs[0][a - 1], refs[1][b - 1], refs[1][0]])
        assert_logits_close(got, ref, dtype, f"{name} step {i} prompts of {a} and {b}")
        for k in range(2):
            got = eng.step([(slots[0], [reqs[0][a + k]]), (slots[1], [reqs[1][b + k]])])
            ref = torch.stack([refs[0][a + k], refs[1][b + k]])
            assert_logits_close(got, ref, dtype, f"{name} step {i} token {k} after the prompts")
        for s in slots:
            eng.end_sequence(s)
    graphs = [g for key, g in eng._prompt_graphs.items() if key[0] == "prompts"]
    assert len(graphs) == 1 and graphs[0].graph is not None and graphs[0].calls == len(lens)
    # (the single-token steps in between were recorded too, as one step of two sequences)
    tokens = [g for key, g in eng._prompt_graphs.items() if key[0] == "tokens"]
    assert len(tokens) == 1 and tokens[0].graph is not None and tokens[0].calls == 2 * len(lens)
    for s in held:
        eng.end_sequence(s)
    assert eng.cache.pages_in_use() == 0


def test_recorded_prompt_steps_can_be_switched_off_and_are_few(model_dirs):
    cfg = CONFIGS["A"]
    eng = _engine(model_dirs, "A", "bfloat16", 64, max_tokens=4096)
    toks = random_prompts(cfg, [40], seed=5)[0]
    ref = plain_logits(toks, model_dirs["A", "bfloat16"], cfg)[-1:]
    eng.prompt_graph_rows = 0
    slot = eng.new_sequence()
    assert_logits_close(eng.step([(slot, toks)]), ref, "bfloat16", "launched one by one")
    eng.end_sequence(slot)
    assert not eng._prompt_graphs
    eng.prompt_graph_rows = 1024
    eng.max_prompt_graphs = 2
    for n_seqs in (1, 2, 3, 1):      # a recording per number of sequences; the oldest goes
        slots = [eng.new_sequence() for _ in range(n_seqs)]
        got = eng.step([(s, toks) for s in slots])
        assert_logits_close(got, ref.expand(n_seqs, -1), "bfloat16", f"{n_seqs} prompts")
        for s in slots:
            eng.end_sequence(s)
        assert len(eng._prompt_graphs) <= 2
    assert [k[2] for k in eng._prompt_graphs] == [3, 1]


@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8), ("C", 16)])
def test_products_of_some_rows_on_the_streaming_tensor_core_kernel(model_dirs, name, page):
    """Every product of 17 to 128 rows through csrc/linear_rows_tc.cu (the engine sends it
    only matrices with very many rows: here the limit is taken away), gated and soft-capped
    epilogues included: 20 prompts in one step, then tokens one by one."""
    cfg = CONFIGS[name]
    eng = _engine(model_dirs, name, "bfloat16", page, max_tokens=4096)
    eng.rt.rows_tc_min_weight_rows = 1
    lens = [3 + (7 * i) % 6 for i in range(20)]          # 3..8 tokens each, about 110 rows
    reqs = random_prompts(cfg, [n + 3 for n in lens], seed=31)
    refs = [plain_logits(t, model_dirs[name, "bfloat16"], cfg) for t in reqs]
    slots = [eng.new_sequence() for _ in reqs]
    from strata_inference_b200.kernels import native
    with native.KernelProfile() as prof:
        got = eng.step([(s, t[:n]) for s, t, n in zip(slots, reqs, lens)])
    assert any(row["name"].startswith("linear_rows_tc") for row in prof.rows())
    ref = torch.stack([refs[i][n - 1] for i, n in enumerate(lens)])
    assert_logits_close(got, ref, "bfloat16", f"{name} 20 prompts")
    for k in range(3):
        got = eng.step([(s, [t[n + k]]) for s, t, n in zip(slots, reqs, lens)])
        ref = torch.stack([refs[i][n + k] for i, n in enumerate(lens)])
        assert_logits_close(got, ref, "bfloat16", f"{name} token {k} of 20 sequences")
    for s in slots:
        eng.end_sequence(s)
    eng.read_back(got)       # (no bounded wait ran out)


def test_a_profiled_step_is_not_recorded(model_dirs):
    """While a kernel profile is being taken, steps are launched kernel by kernel (a
    profile's events cannot go into a CUDA graph); afterwards they are recorded as usual."""
    from strata_inference_b200.engine.profile import profile_step
    cfg = CONFIGS["A"]
    eng = _engine(model_dirs, "A", "bfloat16", 64)
    toks = random_prompts(cfg, [40], seed=5)[0]
    ref = plain_logits(toks, model_dirs["A", "bfloat16"], cfg)[-1:]
    for i in range(3):
        slot = eng.new_sequence()
        got = []
        rows, ms = profile_step(lambda: got.append(eng.step([(slot, toks)])))
        assert any(r["name"].startswith("attention") for r in rows) and ms > 0
        assert_logits_close(got[0], ref, "bfloat16", f"profiled prompt step {i}")
        eng.end_sequence(slot)
    graph = list(eng._prompt_graphs.values())[0]
    assert graph.graph is None
    slot = eng.new_sequence()
    assert_logits_close(eng.step([(slot, toks)]), ref, "bfloat16", "recorded afterwards")
    assert graph.graph is not None
    eng.end_sequence(slot)


def test_tokens_are_fed_on_the_device_only_right_after_the_step_that_sampled_them(model_dirs):
    from strata_inference_b200.engine.engine import StepError
    cfg = CONFIGS["A"]
    eng = _engine(model_dirs, "A", "float32", 64)
    toks = random_prompts(cfg, [30, 30], seed=12)
    ref = [plain_logits(t, model_dirs["A", "float32"], cfg) for t in toks]
    slots = [eng.new_sequence(), eng.new_sequence()]
    eng.step([(s, t[:20]) for s, t in zip(slots, toks)])
    assert not eng.can_feed_back(slots)
    fed = [t[20] for t in toks]
    for i in range(3):          # launched, recorded, replayed: greedy tokens of the plain logits
        out = eng.decode_step(slots, fed)
        want = [int(ref[b][20 + i].argmax()) for b in range(2)]
        fed = eng.read_back(out)
        assert fed == want
        toks = [t[:21 + i] + [w] + t[22 + i:] for t, w in zip(toks, want)]
        ref = [plain_logits(t, model_dirs["A", "float32"], cfg) for t in toks]
    assert eng.can_feed_back(slots) and not eng.can_feed_back(slots[::-1])
    out = eng.decode_step(slots, None)            # fed with `fed`, on the device
    assert eng.read_back(out) == [int(ref[b][23].argmax()) for b in range(2)]
    eng.step([(slots[0], [toks[0][24]])])         # another step in between: no feeding back
    assert not eng.can_feed_back(slots)
    with pytest.raises(StepError, match="right after"):
        eng.decode_step(slots, None)
    for s in slots:
        eng.end_sequence(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_many_short_prompts_in_one_step(model_dirs, dtype):
    """A step of many short prompts (recorded apart from steps with a long prompt: their
    attention runs on the kernel with the cheaper start), then a step with one long prompt
    among short ones, against the plain implementation."""
    name, cfg = "A", CONFIGS["A"]
    eng = _engine(model_dirs, name, dtype, 4, max_tokens=4096)
    eng.rt.short_prompt_tokens = 24          # (the tiny model's prompts are short anyway)
    for rnd, lens in enumerate(([5, 17, 9, 24, 3, 12, 20, 8], [7, 11, 24, 2, 19, 6, 23, 10],
                                [5, 17, 60, 24, 3, 12, 20, 8], [9, 9, 9, 9, 9, 9, 9, 30])):
        reqs = random_prompts(cfg, [n + 1 for n in lens], seed=90 + rnd)
        refs = [plain_logits(t, model_dirs[name, dtype], cfg) for t in reqs]
        slots = [eng.new_sequence() for _ in reqs]
        got = eng.step([(s, t[:n]) for s, t, n in zip(slots, reqs, lens)])
        assert_logits_close(got, torch.stack([r[n - 1] for r, n in zip(refs, lens)]), dtype,
                            f"step {rnd}: prompts of {lens}")
        got = eng.step([(s, [t[n]]) for s, t, n in zip(slots, reqs, lens)])
        assert_logits_close(got, torch.stack([r[n] for r, n in zip(refs, lens)]), dtype,
                            f"step {rnd}: the token after the prompts")
        for s in slots:
            eng.end_sequence(s)
    bounds = {k[4] for k in eng._prompt_graphs if k[0] == "prompts"}
    assert bounds == {None, 24}                      # one recording with the bound, one without
    assert eng.cache.pages_in_use() == 0


def test_single_token_steps_are_recorded_by_length_class(model_dirs):
    """A recorded single-token step divides the attention's work for a class of lengths
    (powers of two from ``first_span``, 512 unless set): sequences that outgrow their class go
    on in the next class's recording, with the plain implementation's logits all along."""
    name, cfg = "C", CONFIGS["C"]
    eng = _engine(model_dirs, name, "float32", 16, max_tokens=1024)
    eng.first_span = 32
    toks = random_prompts(cfg, [150], seed=33)[0]
    ref = plain_logits(toks, model_dirs[name, "float32"], cfg)
    slot = eng.new_sequence()
    eng.step([(slot, toks[:50])])
    choices = []
    for i in range(50, 150):            # crosses 64 and 128 positions
        out = eng.decode_step([slot], [toks[i]])
        choices.append(int(eng.read_back(out)[0]))
        assert_logits_close(eng.last_logits, ref[i:i + 1], "float32", f"position {i}")
    assert choices == [int(ref[i].argmax()) for i in range(50, 150)]
    assert sorted(k[4] for k in eng._graphs) == [64, 128, 256]
    assert all(g.graph is not None for g in eng._graphs.values())
    eng.end_sequence(slot)


@pytest.mark.parametrize("name,page,seed", [("A", 4, 1), ("C", 16, 2), ("B", 8, 3), ("C", 64, 4)])
def test_a_random_schedule_of_steps(model_dirs, name, page, seed):
    """Sequences come and go in a random order of prompt steps, pieces, single-token steps
    through ``step`` and through ``decode_step`` (recorded or not, fed from the host or on
    the device), with other sequences beside them or alone: every logit row that comes back
    is the plain implementation's for that sequence at that position."""
    import random
    rnd = random.Random(seed)
    cfg = CONFIGS[name]
    top = cfg["max_position_embeddings"]
    eng = _engine(model_dirs, name, "float32", page, max_tokens=8 * ((top + 63) // 64) * 64)
    eng.first_span = 32
    room = eng.cache.max_step_tokens()
    live = {}          # slot -> [tokens, reference logits, position]
    checked = 0
    for op in range(70):
        kind = rnd.choice(["new", "new", "piece", "tokens", "tokens", "decode", "decode", "end"])
        if kind == "new" and len(live) < 6:
            fresh = []
            for _ in range(rnd.randint(1, 3)):
                if len(live) + len(fresh) >= 6:
                    break
                toks = random_prompts(cfg, [rnd.randint(top // 2, top - 1)], seed=1000 * seed + op + len(fresh))[0]
                fresh.append((eng.new_sequence(), toks, rnd.randint(1, min(len(toks) - 1, 70))))
            got = eng.step([(s, t[:n]) for s, t, n in fresh])
            for row, (s, t, n) in enumerate(fresh):
                ref = plain_logits(t, model_dirs[name, "float32"], cfg)
                live[s] = [t, ref, n]
                assert_logits_close(got[row:row + 1], ref[n - 1:n], "float32", f"op {op}: prompt of {n}")
                checked += 1
        elif kind == "piece" and live:
            s = rnd.choice(sorted(live))
            t, ref, pos = live[s]
            n = min(rnd.randint(2, 40), len(t) - pos, eng.cache.max_step_tokens(pos))
            if n >= 1:
                got = eng.step([(s, t[pos:pos + n])], want=[[0, n - 1]])
                assert_logits_close(got, torch.stack([ref[pos], ref[pos + n - 1]]), "float32",
                                    f"op {op}: piece of {n} at {pos}")
                live[s][2] = pos + n
                checked += 2
        elif kind in ("tokens", "decode") and live:
            some = [s for s in sorted(live) if live[s][2] < len(live[s][0])]
            some = rnd.sample(some, rnd.randint(1, len(some))) if some else []
            for _ in range(rnd.randint(1, 4)):
                some = [s for s in some if live[s][2] < len(live[s][0])]
                if not some:
                    break
                fed = [live[s][0][live[s][2]] for s in some]
                if kind == "tokens":
                    got = eng.step([(s, [f]) for s, f in zip(some, fed)])
                else:
                    eng.decode_step(some, fed, use_graph=rnd.random() < 0.8)
                    got = eng.last_logits
                ref = torch.stack([live[s][1][live[s][2]] for s in some])
                assert_logits_close(got, ref, "float32", f"op {op}: {kind} for {some}")
                for s in some:
                    live[s][2] += 1
                checked += len(some)
        elif kind == "end" and live:
            s = rnd.choice(sorted(live))
            eng.end_sequence(s)
            del live[s]
        for s in [s for s in live if live[s][2] >= len(live[s][0])]:
            eng.end_sequence(s)
            del live[s]
    for s in list(live):
        eng.end_sequence(s)
    assert checked > 60 and eng.cache.pages_in_use() == 0
    eng.read_back(torch.zeros(1, dtype=torch.int32, device="cuda:0"))      # no bounded wait ran out
