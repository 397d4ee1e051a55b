"""The engine at the layer sizes of Gemma2-2B (hidden 2304, 8 heads of 256 in
4 groups, intermediate 9216, vocabulary 256000) and of Gemma2-27B (hidden 4608,
32 heads of 128 in 16 groups, intermediate 36864), two layers deep, against the
plain implementation: whole prompt, last tokens one by one, unequal batch.
The tiny configurations never reach the code paths that these sizes select
(head size 256, the 16-byte vector paths, the cluster split of the products,
the tensor-memory product for many rows of logits)."""

import os

import pytest
import torch

import plain_gemma2 as plain
from helpers import REL_TOL, plain_weights, random_prompts

pytestmark = pytest.mark.gpu

CFG_2B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 2304, "num_attention_heads": 8,
    "num_key_value_heads": 4, "head_dim": 256, "intermediate_size": 9216, "vocab_size": 256000,
    "rope_theta": 10000.0, "sliding_window": 96, "query_pre_attn_scalar": 256,
    "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 512, "hidden_activation": "gelu_pytorch_tanh",
    "tie_word_embeddings": True,
}
# the layer sizes of Gemma2-27B (32 heads of 128 in 16 groups) with a shorter vocabulary,
# which keeps the plain implementation's 32-bit weights to a few GB
CFG_27B = dict(CFG_2B, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16,
               head_dim=128, intermediate_size=36864, vocab_size=32000, query_pre_attn_scalar=144,
               sliding_window=80)
CONFIGS = {"2b": CFG_2B, "27b": CFG_27B}


def _rel(got, ref):
    got, ref = got.detach().float().cpu(), ref.float()
    return (got - ref).abs().max().item() / ref.abs().max().item()


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    """The model folder, the requests and the plain logits, shared by both types."""
    from strata_inference_b200.weights.random_init import write_random_model
    cfg = CONFIGS[request.param]
    d = str(tmp_path_factory.mktemp("gemma2_%s_sizes" % request.param))
    write_random_model(d, cfg, seed=17, dtype=torch.bfloat16, matrix_std=0.02, norm_std=0.1,
                       device="cuda:0")
    W = {k: v.float() for k, v in plain_weights(d).items()}
    reqs = random_prompts(cfg, [200, 37, 150], seed=18)
    refs = [plain.forward(t, W, cfg, dtype=torch.float32) for t in reqs]
    return d, reqs, refs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_layers_of_real_sizes(model, dtype):
    from strata_inference_b200 import Engine
    d, reqs, refs = model
    tol = REL_TOL[dtype]
    eng = Engine.from_dir(d, dtype=dtype, max_tokens=1024)
    # whole, every position wanted (more than 16 rows of logits)
    s = eng.new_sequence()
    got = eng.step([(s, reqs[0])], want=[list(range(len(reqs[0])))])
    eng.end_sequence(s)
    assert _rel(got, refs[0]) <= tol, f"whole prompt: {_rel(got, refs[0]):.2e}"
    # prefix, then the last 32 tokens one by one (crosses the window of 96 and a page edge)
    s = eng.new_sequence()
    cut = len(reqs[0]) - 32
    outs = [eng.step([(s, reqs[0][:cut])])]
    for t in reqs[0][cut:]:
        outs.append(eng.step([(s, [t])]))
    eng.end_sequence(s)
    err = _rel(torch.cat(outs), refs[0][cut - 1:])
    assert err <= tol, f"last 32 one by one: {err:.2e}"
    # an unequal batch, then 5 single-token steps; the short request ends after 3
    prompt = [120, 30, 100]
    slots = [eng.new_sequence() for _ in reqs]
    got = eng.step([(sl, r[:p]) for sl, r, p in zip(slots, reqs, prompt)])
    ref = torch.stack([f[p - 1] for f, p in zip(refs, prompt)])
    assert _rel(got, ref) <= tol, f"batch prompts: {_rel(got, ref):.2e}"
    live = [0, 1, 2]
    for k in range(5):
        if k == 3:
            eng.end_sequence(slots[1])
            live = [0, 2]
        got = eng.step([(slots[i], [reqs[i][prompt[i] + k]]) for i in live])
        ref = torch.stack([refs[i][prompt[i] + k] for i in live])
        assert _rel(got, ref) <= tol, f"batch step {k}: {_rel(got, ref):.2e}"
    for i in live:
        eng.end_sequence(slots[i])
    assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_of_4096_at_real_sizes(tmp_path, dtype):
    """Two layers at Gemma2-2B sizes with the real window of 4096: a 4 100-token prompt (the
    paired tcgen05 prompt kernel with a window; the sliding layer's ring of 4 160 positions
    is written around once), then 150 single-token steps that take the ring over its end.
    The plain implementation runs on the GPU here (its code is the same; 4 250 x 4 250 scores
    per head are too slow on the host)."""
    from strata_inference_b200 import Engine
    from strata_inference_b200.weights.random_init import write_random_model
    cfg = dict(CFG_2B, vocab_size=32000, sliding_window=4096, max_position_embeddings=8192)
    d = str(tmp_path / "gemma2_window")
    write_random_model(d, cfg, seed=3, dtype=torch.bfloat16, matrix_std=0.02, norm_std=0.1,
                       device="cuda:0")
    toks = random_prompts(cfg, [4250], seed=4)[0]
    with torch.no_grad(), torch.device("cuda"):
        W = {k: v.float().cuda() for k, v in plain_weights(d).items()}
        ref = plain.forward(toks, W, cfg, dtype=torch.float32).cpu()
    del W
    eng = Engine.from_dir(d, dtype=dtype, max_tokens=8192)
    s = eng.new_sequence()
    outs = [eng.step([(s, toks[:4100])], want=[[4098, 4099]])]
    for t in toks[4100:]:
        outs.append(eng.step([(s, [t])]))
    eng.end_sequence(s)
    err = _rel(torch.cat(outs), ref[4098:])
    assert err <= REL_TOL[dtype], f"window of 4096, {dtype}: {err:.2e}"


# ---------------------------------------------------------------- the whole Gemma2-2B shape

CFG_2B_FULL = dict(CFG_2B, num_hidden_layers=26, sliding_window=4096, max_position_embeddings=8192)


def _stored_on_device(cfg, seed):
    """The stored tensors that `seed` names, drawn on the device (weights are inputs of the
    plain implementation; the generator is checked against its host formula elsewhere)."""
    from strata_inference_b200.config.registry import spec_from_config
    from strata_inference_b200.engine.model import expected_tensors
    from strata_inference_b200.weights.random_init import random_tensors
    _, spec = spec_from_config(cfg)
    return random_tensors(expected_tensors(spec), seed, torch.bfloat16, "cuda:0")


@pytest.fixture(scope="module")
def full_2b():
    cfg = CFG_2B_FULL
    reqs = random_prompts(cfg, [320, 70, 200, 45, 130, 90], seed=28)
    torch.backends.cuda.matmul.allow_tf32 = False
    with torch.no_grad(), torch.device("cuda"):
        W = {k: v.float() for k, v in _stored_on_device(cfg, 5).items()}
        refs = [plain.forward(t, W, cfg, dtype=torch.float32).cpu() for t in reqs]
    del W
    torch.cuda.empty_cache()
    return cfg, reqs, refs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_26_layers_of_the_2b_shape(full_2b, dtype):
    """Gemma2-2B's configuration at full depth (26 layers, vocabulary 256 000, window 4 096,
    context 8 192), the model that seed 5 names: a request whole with every position wanted;
    its last 32 tokens one by one; an unequal batch whose shortest request leaves first; a
    second batch on the slots that the first gave back."""
    from strata_inference_b200 import Engine
    cfg, reqs, refs = full_2b
    tol = REL_TOL[dtype]
    eng = Engine.from_random(cfg, 5, dtype=dtype, store="bfloat16", max_tokens=2048, max_slots=4)
    assert len(eng.model.blocks) == 26 and sum(len(g.entries) for g in eng.cache.groups) == 26
    s = eng.new_sequence()
    got = eng.step([(s, reqs[0])], want=[list(range(len(reqs[0])))])
    eng.end_sequence(s)
    assert _rel(got, refs[0]) <= tol, f"whole request: {_rel(got, refs[0]):.2e}"
    s = eng.new_sequence()
    cut = len(reqs[0]) - 32
    outs = [eng.step([(s, reqs[0][:cut])])]
    for t in reqs[0][cut:]:
        outs.append(eng.step([(s, [t])]))
    eng.end_sequence(s)
    err = _rel(torch.cat(outs), refs[0][cut - 1:])
    assert err <= tol, f"last 32 one by one: {err:.2e}"

    def batch(which, prompt, steps, tag):
        slots = [eng.new_sequence() for _ in which]
        got = eng.step([(sl, reqs[i][:p]) for sl, i, p in zip(slots, which, prompt)])
        ref = torch.stack([refs[i][p - 1] for i, p in zip(which, prompt)])
        assert _rel(got, ref) <= tol, f"{tag} prompts: {_rel(got, ref):.2e}"
        live = list(range(len(which)))
        for k in range(steps):
            for j in list(live):
                if prompt[j] + k >= len(reqs[which[j]]):        # used up: it leaves
                    eng.end_sequence(slots[j])
                    live.remove(j)
            got = eng.step([(slots[j], [reqs[which[j]][prompt[j] + k]]) for j in live])
            ref = torch.stack([refs[which[j]][prompt[j] + k] for j in live])
            assert _rel(got, ref) <= tol, f"{tag} step {k}: {_rel(got, ref):.2e}"
        for j in live:
            eng.end_sequence(slots[j])
        return slots
    first = batch([0, 1, 2, 3], [300, 60, 150, 40], 12, "batch 1")     # request 3 leaves after 5
    assert eng.cache.pages_in_use() == 0
    second = batch([4, 5, 1], [100, 85, 30], 8, "batch 2")             # request 5 leaves after 5
    assert set(second) <= set(first) and eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_twenty_requests_at_2b_sizes(dtype):
    """Two layers at Gemma2-2B sizes: 20 prompts of 100 to 1 600 tokens in one step, then six
    single-token steps through the captured step (more rows than the weight-streaming
    kernels take, prompts across several blocks of the prompt-attention kernel)."""
    from strata_inference_b200 import Engine
    cfg = dict(CFG_2B, vocab_size=32000, sliding_window=512, max_position_embeddings=2048)
    g = torch.Generator().manual_seed(31)
    lens = [100] + torch.randint(100, 1601, (18,), generator=g).tolist() + [1600]
    reqs = random_prompts(cfg, [n + 6 for n in lens], seed=32)
    torch.backends.cuda.matmul.allow_tf32 = False
    with torch.no_grad(), torch.device("cuda"):
        W = {k: v.float() for k, v in _stored_on_device(cfg, 33).items()}
        refs = [plain.forward(t, W, cfg, dtype=torch.float32)[n - 1:].cpu()
                for t, n in zip(reqs, lens)]
    del W
    eng = Engine.from_random(cfg, 33, dtype=dtype, store="bfloat16",
                             max_tokens=sum(lens) + 64 * 21 + 256)
    slots = [eng.new_sequence() for _ in reqs]
    got = eng.step([(s, r[:n]) for s, r, n in zip(slots, reqs, lens)])
    tol = REL_TOL[dtype]
    err = _rel(got, torch.stack([f[0] for f in refs]))
    assert err <= tol, f"20 prompts: {err:.2e}"
    for k in range(6):
        eng.decode_step(slots, [r[n + k] for r, n in zip(reqs, lens)])
        err = _rel(eng.last_logits, torch.stack([f[k + 1] for f in refs]))
        assert err <= tol, f"20 sequences, captured step {k}: {err:.2e}"
    for s in slots:
        eng.end_sequence(s)
    assert eng.cache.pages_in_use() == 0


def test_eight_prompts_of_128_to_4096_at_9b_sizes():
    """Two layers at Gemma2-9B sizes (hidden 3584, 16 heads of 256 in 8 groups, intermediate
    14 336, window 4 096) in bfloat16: an unequal batch of 8 prompts of 128 to 4 096 tokens
    in one step, then four tokens each."""
    from strata_inference_b200 import Engine
    cfg = dict(CFG_2B, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8,
               head_dim=256, intermediate_size=14336, vocab_size=32000, sliding_window=4096,
               max_position_embeddings=8192)
    lens = [128, 4096, 700, 2048, 333, 4000, 1500, 129]
    reqs = random_prompts(cfg, [n + 4 for n in lens], seed=41)
    torch.backends.cuda.matmul.allow_tf32 = False
    with torch.no_grad(), torch.device("cuda"):
        W = {k: v.float() for k, v in _stored_on_device(cfg, 6).items()}
        refs = [plain.forward(t, W, cfg, dtype=torch.float32)[n - 1:].cpu()
                for t, n in zip(reqs, lens)]
    del W
    eng = Engine.from_random(cfg, 6, dtype="bfloat16", max_tokens=sum(lens) + 64 * 10)
    slots = [eng.new_sequence() for _ in reqs]
    got = eng.step([(s, r[:n]) for s, r, n in zip(slots, reqs, lens)])
    tol = REL_TOL["bfloat16"]
    err = _rel(got, torch.stack([f[0] for f in refs]))
    assert err <= tol, f"8 prompts: {err:.2e}"
    for k in range(4):
        eng.decode_step(slots, [r[n + k] for r, n in zip(reqs, lens)])
        err = _rel(eng.last_logits, torch.stack([f[k + 1] for f in refs]))
        assert err <= tol, f"8 sequences, step {k}: {err:.2e}"
    for s in slots:
        eng.end_sequence(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_at_real_sizes_one_step_ahead_of_the_host(model, dtype):
    """Generation through the entry point at real layer sizes and vocabulary, with the
    reference's default sampling options (temperature 0.8, top-k 40, top-p 0.95, the list
    path of the sampling kernel) and greedy: the loop that keeps the device a step ahead
    gives the tokens of the loop that waits for every step; in 32-bit the greedy tokens are
    the plain implementation's."""
    from strata_inference_b200 import GenerationConfig, GenerationEngine, SamplingConfig
    d, reqs, refs = model
    cfg = [c for c in CONFIGS.values() if c["vocab_size"] == refs[0].shape[1]][0]
    gen = GenerationEngine.from_dir(d, dtype=dtype, max_tokens=2048)
    prompts = [reqs[0][:150], reqs[1][:20], reqs[2][:90]]
    for sampling in (SamplingConfig(temperature=0.8, top_k=40, top_p=0.95, seed=3), SamplingConfig()):
        waited = gen.generate(prompts, GenerationConfig(max_tokens=10, sampling=sampling, look_ahead=False))
        ahead = gen.generate(prompts, GenerationConfig(max_tokens=10, sampling=sampling, look_ahead=True))
        assert [o.token_ids for o in waited] == [o.token_ids for o in ahead]
        assert all(len(o.token_ids) == 10 or o.stop_reason == "eos" for o in ahead)
    if dtype == "float32":
        W = {k: v.float() for k, v in plain_weights(d).items()}
        for p, o in zip(prompts[1:2], ahead[1:2]):       # the short request: 10 plain steps
            seq = list(p)
            for tok in o.token_ids:
                logits = plain.forward(seq, W, cfg, dtype=torch.float32)[-1]
                top = torch.topk(logits, 2).values
                assert int(logits.argmax()) == tok or float(top[0] - top[1]) < 1e-4 * float(top[0].abs())
                seq.append(tok)
    assert gen.engine.cache.pages_in_use() == 0


def test_a_prompt_that_comes_in_pieces_at_real_sizes(model):
    """A request continued in pieces of 64 and 37 tokens (the windowed layer's ring wraps),
    alone and beside a second request that goes on token by token: the pieces attend
    through the prompt kernel over a packed copy of what the sequence holds."""
    from strata_inference_b200 import Engine
    from strata_inference_b200.kernels import native
    d, reqs, refs = model
    tol = REL_TOL["bfloat16"]
    eng = Engine.from_dir(d, dtype="bfloat16", max_tokens=2048, max_continuation=64)
    s = eng.new_sequence()
    outs, at = [], 0
    with native.KernelProfile() as prof:
        for piece in (40, 64, 64):
            outs.append(eng.step([(s, reqs[0][at:at + piece])], want=[list(range(piece))]))
            at += piece
    if os.environ.get("SIB_PREFILL_TCGEN05") != "0":       # (the switch also takes this path away)
        assert any(r["name"] == "gather_kv_rows" for r in prof.rows())
    err = _rel(torch.cat(outs), refs[0][:at])
    assert err <= tol, f"pieces of one request: {err:.2e}"
    # a second request beside it: its prompt, then single tokens while the first goes on in pieces
    s2 = eng.new_sequence()
    eng.step([(s2, reqs[2][:50])])
    got = eng.step([(s, reqs[0][at:]), (s2, [reqs[2][50]])], want=[[len(reqs[0]) - at - 1], [0]])
    ref = torch.stack([refs[0][-1], refs[2][50]])
    assert _rel(got, ref) <= tol, f"a piece beside a single token: {_rel(got, ref):.2e}"
    eng.end_sequence(s)
    eng.end_sequence(s2)
    assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype,seed", [("bfloat16", 1), ("bfloat16", 2), ("float32", 3)])
def test_a_random_schedule_at_real_sizes(model, dtype, seed):
    """The three requests start, go on in pieces, token by token through ``step`` and through
    recorded steps, end and start again in a random order, alone or beside each other: every
    row of logits that comes back is the plain implementation's.  (At these sizes the steps
    run the tcgen05 prompt attention as a list and over gathered pieces, the mma.sync prompt
    attention for short prompts, the decode attention with its splits, the weight-streaming
    products and the library's.)"""
    import random
    from strata_inference_b200 import Engine
    d, reqs, refs = model
    tol = REL_TOL[dtype]
    rnd = random.Random(seed)
    eng = Engine.from_dir(d, dtype=dtype, max_tokens=2048, max_continuation=64)
    eng.first_span = 64
    live, worst, checked = {}, 0.0, 0          # request -> [slot, position]

    def check(got, rows, what):
        nonlocal worst, checked
        ref = torch.stack([refs[i][p] for i, p in rows])
        err = _rel(got, ref)
        worst = max(worst, err)
        checked += len(rows)
        assert err <= tol, f"{what}: {err:.2e}"

    for op in range(90):
        kind = rnd.choice(["new", "piece", "tokens", "tokens", "decode", "decode", "end"])
        idle = [i for i in range(3) if i not in live]
        if kind == "new" and idle:
            some = rnd.sample(idle, rnd.randint(1, len(idle)))
            cut = {i: rnd.randint(1, len(reqs[i]) - 2) for i in some}
            for i in some:
                live[i] = [eng.new_sequence(), cut[i]]
            got = eng.step([(live[i][0], reqs[i][:cut[i]]) for i in some])
            check(got, [(i, cut[i] - 1) for i in some], f"op {op}: prompts {cut}")
        elif kind == "piece" and live:
            i = rnd.choice(sorted(live))
            s, pos = live[i]
            n = min(rnd.randint(2, 64), len(reqs[i]) - pos, eng.cache.max_step_tokens(pos))
            if n >= 1:
                got = eng.step([(s, reqs[i][pos:pos + n])], want=[[0, n - 1]])
                check(got, [(i, pos), (i, pos + n - 1)], f"op {op}: piece of {n} at {pos}")
                live[i][1] = pos + n
        elif kind in ("tokens", "decode") and live:
            some = rnd.sample(sorted(live), rnd.randint(1, len(live)))
            for _ in range(rnd.randint(1, 5)):
                some = [i for i in some if live[i][1] < len(reqs[i])]
                if not some:
                    break
                fed = [reqs[i][live[i][1]] for i in some]
                if kind == "tokens":
                    got = eng.step([(live[i][0], [f]) for i, f in zip(some, fed)])
                else:
                    eng.decode_step([live[i][0] for i in some], fed, use_graph=rnd.random() < 0.8)
                    got = eng.last_logits
                check(got, [(i, live[i][1]) for i in some], f"op {op}: {kind} for {some}")
                for i in some:
                    live[i][1] += 1
        elif kind == "end" and live:
            i = rnd.choice(sorted(live))
            eng.end_sequence(live.pop(i)[0])
        for i in [i for i in live if live[i][1] >= len(reqs[i])]:
            eng.end_sequence(live.pop(i)[0])
    for i in list(live):
        eng.end_sequence(live.pop(i)[0])
    assert checked > 25 and eng.cache.pages_in_use() == 0
    eng.read_back(torch.zeros(1, dtype=torch.int32, device="cuda:0"))
