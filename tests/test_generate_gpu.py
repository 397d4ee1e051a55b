"""Generation through the entry points (Python API, command line, trace
replay) against the plain implementation."""

import json
import os
import struct
import subprocess
import sys

import pytest
import torch

import plain_gemma2 as plain
from helpers import (CONFIGS, SHARPEN, assert_logits_close, eos_list, make_model_dir, plain_logits, plain_weights,
                     random_prompts)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: make_model_dir(str(tmp_path_factory.mktemp(f"gen_{name}")), cfg, seed=30 + i)
            for i, (name, cfg) in enumerate(CONFIGS.items())}


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("use_graph", [True, False])
def test_greedy_generation_matches_plain(model_dirs, name, use_graph):
    """BASELINE's workloads: unequal prompts, greedy steps, 32-bit: the same tokens as
    the plain implementation that recomputes every step from the first token."""
    from strata_inference_b200 import GenerationConfig, GenerationEngine
    cfg = CONFIGS[name]
    lengths = [5, 9, 13] if name == "A" else [20, 3]
    steps = 8 if name == "A" else 12
    prompts = random_prompts(cfg, lengths, seed=1)
    eng = GenerationEngine.from_dir(model_dirs[name], dtype="float32", max_tokens=512,
                                    use_graph=use_graph)
    outs = eng.generate(prompts, GenerationConfig(max_tokens=steps))
    W = plain_weights(model_dirs[name])
    for p, o in zip(prompts, outs):
        want, reason = plain.generate(p, W, cfg, steps, stop_tokens=eos_list(cfg))
        assert o.token_ids == want and o.stop_reason == reason and o.prompt_tokens == len(p)
    assert eng.engine.cache.pages_in_use() == 0


def test_sampled_generation_alone_and_in_batch(model_dirs):
    """Temperature sampling with fixed seeds: a request draws the same tokens
    alone, in a batch, and in the plain implementation."""
    from strata_inference_b200 import GenerationConfig, GenerationEngine, SamplingConfig
    name, cfg = "B", CONFIGS["B"]
    prompts = random_prompts(cfg, [20, 3, 11], seed=3)
    conf = GenerationConfig(max_tokens=12, sampling=SamplingConfig(temperature=0.8, seed=4))
    eng = GenerationEngine.from_dir(model_dirs[name], dtype="float32", max_tokens=512)
    together = eng.generate(prompts, conf)
    alone = [eng.generate([p], conf)[0] for p in prompts]
    W = plain_weights(model_dirs[name])
    for p, t, a in zip(prompts, together, alone):
        assert t.token_ids == a.token_ids
        want, _ = plain.generate(p, W, cfg, 12, stop_tokens=eos_list(cfg), temperature=0.8, seed=4)
        assert t.token_ids == want
    seeded = eng.generate(prompts, conf, seeds=[4, 5, 6])
    assert seeded[0].token_ids == together[0].token_ids
    assert seeded[1].token_ids != together[1].token_ids or seeded[2].token_ids != together[2].token_ids


def test_stop_tokens_context_end_and_batches_one_after_another(model_dirs):
    from strata_inference_b200 import GenerationConfig, GenerationEngine
    name, cfg = "B", CONFIGS["B"]
    W = plain_weights(model_dirs[name])
    prompts = random_prompts(cfg, [7, 30, 2, 50, 12, 5], seed=5)
    # a cache too small for all six at once: several batches, slots used again
    eng = GenerationEngine.from_dir(model_dirs[name], dtype="float32", max_tokens=192)
    free = plain.generate(prompts[0], W, cfg, 10)[0]
    stop = free[4]
    conf = GenerationConfig(max_tokens=-1, stop_tokens=[stop])
    outs = eng.generate(prompts, conf)
    for p, o in zip(prompts, outs):
        want, reason = plain.generate(p, W, cfg, 10 ** 6, stop_tokens=[stop] + eos_list(cfg))
        assert o.token_ids == want and o.stop_reason == reason
        assert stop not in o.token_ids
    assert {o.stop_reason for o in outs} <= {"eos", "context_length"}
    assert any(o.stop_reason == "context_length" for o in outs)
    assert eng.engine.cache.pages_in_use() == 0


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_one_step_ahead_of_the_host_gives_the_same_tokens(model_dirs, temperature):
    """The loop keeps the device one step ahead (a step is fed with the tokens of the step
    before on the device, before the host has read them): the same tokens, stop reasons and
    freed slots as with every step waited for, also where sequences end at different steps."""
    from strata_inference_b200 import GenerationConfig, GenerationEngine, SamplingConfig
    name, cfg = "B", CONFIGS["B"]
    prompts = random_prompts(cfg, [7, 30, 2, 21, 12, 5], seed=8)
    eng = GenerationEngine.from_dir(model_dirs[name], dtype="float32", max_tokens=512)
    sampling = SamplingConfig(temperature=temperature, seed=9)
    waited = eng.generate(prompts, GenerationConfig(max_tokens=-1, sampling=sampling, look_ahead=False))
    stop = waited[1].token_ids[6]
    fed = []
    step = eng.engine.decode_step

    def counting(slots, tokens, *a, **kw):
        fed.append(tokens is None)
        return step(slots, tokens, *a, **kw)
    eng.engine.decode_step = counting
    for limit in (-1, 9):
        conf = dict(max_tokens=limit, stop_tokens=[stop], sampling=sampling)
        a = eng.generate(prompts, GenerationConfig(look_ahead=False, **conf))
        assert not any(fed)
        b = eng.generate(prompts, GenerationConfig(look_ahead=True, **conf))
        assert sum(fed) >= 4      # steps that took their tokens on the device
        del fed[:]
        assert [(o.token_ids, o.stop_reason) for o in a] == [(o.token_ids, o.stop_reason) for o in b]
        assert len({o.stop_reason for o in a}) > 1
        assert eng.engine.cache.pages_in_use() == 0


def test_bfloat16_generation_is_deterministic_and_every_choice_is_near_the_plain_best(model_dirs):
    from helpers import assert_greedy_choices_close
    from strata_inference_b200 import GenerationConfig, GenerationEngine
    cfg = CONFIGS["C"]
    prompts = random_prompts(cfg, [33, 4, 70], seed=6)
    eng = GenerationEngine.from_dir(model_dirs["C"], dtype="bfloat16", max_tokens=1024)
    a = eng.generate(prompts, GenerationConfig(max_tokens=40))
    b = eng.generate(prompts, GenerationConfig(max_tokens=40))
    for r, (x, y) in enumerate(zip(a, b)):
        first = next((i for i, (u, v) in enumerate(zip(x.token_ids, y.token_ids)) if u != v), None)
        assert x.token_ids == y.token_ids, f"request {r}: the two runs differ from token {first} on"
    assert all(len(o.token_ids) == 40 for o in a)
    W = plain_weights(model_dirs["C"])
    for r, (p, o) in enumerate(zip(prompts, a)):
        assert_greedy_choices_close(p, o.token_ids, W, cfg, "bfloat16", f"request {r}")


def test_command_line_json(model_dirs):
    cfg = CONFIGS["A"]
    prompt = random_prompts(cfg, [6], seed=7)[0]
    cmd = [sys.executable, "-m", "strata_inference_b200.cli", "-m", model_dirs["A"],
           "--token-ids", ",".join(map(str, prompt)), "-n", "5", "--temp", "0",
           "--dtype", "float32", "--output-format", "json", "--log-disable"]
    r = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout)
    want, reason = plain.generate(prompt, plain_weights(model_dirs["A"]), cfg, 5,
                                  stop_tokens=eos_list(cfg))
    assert out["output_token_ids"] == want and out["stop_reason"] == reason
    assert out["generated_tokens"] == len(want)
    assert set(out["timings"]) >= {"load_ms", "prefill_ms", "decode_ms", "total_ms",
                                   "prefill_tok_per_sec", "decode_tok_per_sec"}
    assert out["config"]["max_tokens"] == 5


def _replay(model_dir, dtype, steps, out_dir, max_tokens):
    """Drive bin/trace_run the way a user does: one line in, one 'done' out."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
           "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=ROOT)
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        line = p.stdout.readline().strip()
        assert line == f"done {s['step']}", f"trace_run answered {line!r}"
    p.stdin.close()
    assert p.wait(timeout=600) == 0


def _read(out_dir, step, vocab):
    with open(os.path.join(out_dir, f"{step}.f32"), "rb") as f:
        raw = f.read()
    n = len(raw) // 4
    return torch.tensor(struct.unpack(f"<{n}f", raw)).view(-1, vocab)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay(model_dirs, tmp_path, dtype):
    """Whole requests, last tokens one by one, and an unequal batch whose
    shorter request ends earlier, then a second batch on the freed cache."""
    name, cfg = "A", CONFIGS["A"]
    V = cfg["vocab_size"]
    model_dir = make_model_dir(str(tmp_path / "model"), cfg, seed=40, sharpen=SHARPEN[dtype])
    reqs = random_prompts(cfg, [70, 40, 90], seed=8)
    refs = [plain_logits(t, model_dir, cfg) for t in reqs]
    a, b, c = reqs
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a, "want": list(range(len(a)))}], "end": ["a"]},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:30], "want": [29]}], "end": []},
    ]
    for i in range(30, 40):
        steps.append({"step": len(steps), "entries": [{"id": "b", "tokens": [b[i]], "want": [0]}],
                      "end": ["b"] if i == 39 else []})
    first_batch = len(steps)
    steps.append({"step": first_batch, "entries": [{"id": "a2", "tokens": a[:50], "want": [49]},
                                                    {"id": "c", "tokens": c[:64], "want": [0, 63]}],
                  "end": []})
    for i in range(20):
        ents = [{"id": "a2", "tokens": [a[50 + i]], "want": [0]}]
        ents.append({"id": "c", "tokens": [c[64 + i]], "want": [] if i % 2 else [0]})
        steps.append({"step": len(steps), "entries": ents, "end": ["a2"] if i == 19 else []})
    tail = len(steps)
    for i in range(84, 90):
        steps.append({"step": len(steps), "entries": [{"id": "c", "tokens": [c[i]], "want": [0]}],
                      "end": ["c"] if i == 89 else []})
    out = str(tmp_path / "out")
    _replay(model_dir, dtype, steps, out, max_tokens=256)
    assert_logits_close(_read(out, 0, V), refs[0], dtype, "whole request")
    assert_logits_close(_read(out, 1, V), refs[1][29:30], dtype, "prefix")
    for k, i in enumerate(range(30, 40)):
        assert_logits_close(_read(out, 2 + k, V), refs[1][i:i + 1], dtype, f"b token {i}")
    assert_logits_close(_read(out, first_batch, V),
                        torch.stack([refs[0][49], refs[2][0], refs[2][63]]), dtype, "batch prompts")
    for i in range(20):
        want = [refs[0][50 + i]] + ([] if i % 2 else [refs[2][64 + i]])
        assert_logits_close(_read(out, first_batch + 1 + i, V), torch.stack(want), dtype,
                            f"batch step {i}")
    for k, i in enumerate(range(84, 90)):
        assert_logits_close(_read(out, tail + k, V), refs[2][i:i + 1], dtype, f"c token {i}")


def test_command_line_profile_prints_a_table_per_kernel(model_dirs):
    """--profile: per-token times and, for one prompt step and one captured single-token
    step, the device time of every kernel class with its share of the peak."""
    prompt = random_prompts(CONFIGS["B"], [20], seed=8)[0]
    cmd = [sys.executable, "-m", "strata_inference_b200.cli", "-m", model_dirs["B"],
           "--token-ids", ",".join(map(str, prompt)), "-n", "4", "--temp", "0", "--profile",
           "--no-display-prompt"]
    r = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr
    err = r.stderr
    assert err.count("[profile] request 0 token") == 4
    assert "[profile] prompt step, 20 tokens" in err and "single-token step near position" in err
    table = [l.split() for l in err.splitlines() if l.startswith("[profile] attention")]
    assert len(table) >= 2 and all(float(row[-1]) >= 0.0 for row in table)
    for kernel in ("add_rms_norm", "rms_norm", "embed_rows", "sample_rows", "(between kernels)"):
        assert kernel in err, kernel
