#!/usr/bin/env python3
"""Decode and prefill throughput of strata_inference_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  The run: Gemma2-2B's layer sizes with random bfloat16
weights, a batch of 8 sequences that each hold close to the 8,192-token
context; a "step" is one decode step (one new token per sequence).

* ``value``: decoded tokens per second: five blocks of K steps each are timed on the
  device with CUDA events around the replayed step graphs (tokens are fed from the
  host each step; the result is not read back); the median block counts, the
  fastest and slowest are reported as ``spread_ms``.
* ``e2e``: the same through the Python entry point ``GenerationEngine.generate``:
  host token lists in, host token lists out, wall clock over the decode steps.  Every
  step copies its integers from pinned host memory and its sampled tokens are read on
  the host; the loop keeps the device one step ahead of the host (a step takes the
  tokens of the step before on the device, before the host has read and judged them),
  which ``steps_ahead_of_host`` records.
* ``prefill``: one 2,048-token prompt through ``Engine.step``.
* ``roofline``: bytes a decode step has to read (every weight once, the keys and
  values each live sequence's layers attend to) / its time / the measured copy
  bandwidth.
* ``points``: decoded tokens per second at batch 1 and 64, and at batch 8 of the
  Gemma2-9B and Gemma2-27B shapes at full depth (same context) when they fit.

Between timed steps nothing flushes L2: each step reads 5 GB of weights and more
of cache, against 126 MB of L2.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s at batch 8 (BF16, one B200, Gemma2-2B shape, context 8192)"


def baseline_config():
    """Layer sizes of BASELINE.json's configs[2] (Gemma2-2B shape)."""
    return {
        "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
        "num_hidden_layers": 26, "hidden_size": 2304, "num_attention_heads": 8,
        "num_key_value_heads": 4, "head_dim": 256, "intermediate_size": 9216,
        "vocab_size": 256000, "rope_theta": 10000.0, "sliding_window": 4096,
        "query_pre_attn_scalar": 256, "attn_logit_softcapping": 50.0,
        "final_logit_softcapping": 30.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 8192,
        "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True,
    }


# Other shapes of the same architecture (BASELINE.json's configs[3] and [4]); the default
# run and the recorded line are the 2B shape.
SHAPES = {
    "2b": {},
    "9b": {"num_hidden_layers": 42, "hidden_size": 3584, "num_attention_heads": 16,
           "num_key_value_heads": 8, "head_dim": 256, "intermediate_size": 14336,
           "query_pre_attn_scalar": 256},
    "27b": {"num_hidden_layers": 46, "hidden_size": 4608, "num_attention_heads": 32,
            "num_key_value_heads": 16, "head_dim": 128, "intermediate_size": 36864,
            "query_pre_attn_scalar": 144},
}


def kv_bytes_per_sequence(cfg, context):
    """Bytes of cache one sequence of `context` tokens holds (bfloat16 keys and values)."""
    per_token = cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * 2
    total = 0
    for i in range(cfg["num_hidden_layers"]):
        kept = min(context, cfg["sliding_window"] + 64) if i % 2 == 0 else context
        total += kept * per_token
    return total


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.rows)}


def fill_context(engine, slots, n_tokens):
    """Give each slot ``n_tokens`` positions of random keys and values (what a
    prompt of that length would leave, without running it)."""
    import torch
    engine.cache.reserve([(s, n_tokens) for s in slots])
    for s in slots:
        engine.cache.advance(s, n_tokens)
    engine.cache.sync_tables()


def randomize_pools(engine):
    import torch
    g = torch.Generator(device=engine.device).manual_seed(11)
    for grp in engine.cache.groups:
        for pool in (grp.k, grp.v):
            for layer in range(pool.shape[0]):
                pool[layer].normal_(0.0, 0.5, generator=g)


def kv_bytes_per_step(engine, lengths):
    """Bytes of keys and values one decode step reads for sequences of these lengths."""
    total = 0
    for grp in engine.cache.groups:
        per_token = 2 * grp.need.n_kv_heads * grp.need.head_dim * grp.k.element_size()
        for n in lengths:
            seen = min(n, grp.need.window) if grp.need.window else n
            total += len(grp.entries) * seen * per_token
    return total


BLOCKS = 5      # timed blocks of K steps; the median block is the number


def time_decode(engine, batch, context, steps, warmup, blocks=BLOCKS):
    """ms per decode step (device time; median, fastest and slowest block of ``steps``) for
    ``batch`` sequences near ``context`` positions."""
    import torch
    total = blocks * steps + warmup + 2
    start_len = context - total
    slots = [engine.new_sequence() for _ in range(batch)]
    fill_context(engine, slots, start_len)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, engine.vocab_size, (total, batch), generator=g).tolist()
    for i in range(warmup + 2):            # eager, capture, then replays
        engine.decode_step(slots, toks[i])
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    marks[0].record()
    at = warmup + 2
    for b in range(blocks):
        for i in range(steps):
            engine.decode_step(slots, toks[at + i])
        at += steps
        marks[b + 1].record()
    torch.cuda.synchronize()
    engine.kernel_watch.fetch()
    torch.cuda.synchronize()
    engine.kernel_watch.check()            # a kernel that gave up would make the number void
    per_step = sorted(marks[b].elapsed_time(marks[b + 1]) / steps for b in range(blocks))
    lengths = [engine.length(s) for s in slots]
    graph = engine.recorded_step(batch)
    launches = graph.launches_per_step
    for s in slots:
        engine.end_sequence(s)
    return per_step[len(per_step) // 2], lengths, launches, (per_step[0], per_step[-1])


def time_prefill(engine, n_tokens, reps=5):
    import torch
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, engine.vocab_size, (n_tokens,), generator=g).tolist()
    times = []
    for i in range(reps + 2):
        slot = engine.new_sequence()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        engine.step([(slot, toks)])
        end.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(begin.elapsed_time(end))
        engine.end_sequence(slot)
    engine.kernel_watch.fetch()
    torch.cuda.synchronize()
    engine.kernel_watch.check()
    return statistics.median(times)


def prefill_flops(cfg, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd, L = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                      cfg["num_hidden_layers"])
    per_layer = 2 * T * H * (nh + 2 * nkv) * hd + 2 * T * nh * hd * H + 3 * 2 * T * H * I
    attn = 0
    for i in range(L):
        w = cfg["sliding_window"] if i % 2 == 0 else 0
        pairs = sum(min(p + 1, w) if w else p + 1 for p in range(T))
        attn += 4 * pairs * nh * hd
    return L * per_layer + attn + 2 * H * V          # logits of the last row only


def run_ours(args):
    import torch
    from strata_inference_b200 import GenerationConfig, GenerationEngine

    cfg = baseline_config()
    cfg.update(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    context, batch = args.context, args.batch
    peaks = measured_peaks()
    point_batches = [] if args.no_points else [1, 64]
    weights_estimate = 2 * (cfg["vocab_size"] * cfg["hidden_size"] + cfg["num_hidden_layers"] * (
        cfg["hidden_size"] * (2 * cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"])
        * cfg["head_dim"] + 3 * cfg["hidden_size"] * cfg["intermediate_size"]))
    # a point whose cache would not fit beside the weights is left out
    point_batches = [b for b in point_batches
                     if weights_estimate + b * kv_bytes_per_sequence(cfg, context) < 150e9]
    biggest = max([batch] + point_batches)
    gen = GenerationEngine.from_random(cfg, seed=5, dtype="bfloat16", ctx=context,
                                       max_tokens=biggest * context, max_slots=biggest)
    engine = gen.engine
    randomize_pools(engine)
    weight_bytes = engine.model.weight_bytes()

    with ClockSampler() as clocks:
        ms, lengths, launches, spread = time_decode(engine, batch, context, args.steps,
                                                    args.warmup)
    value = batch * 1e3 / ms
    step_bytes = weight_bytes + kv_bytes_per_step(engine, lengths)
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # (the prompt step is timed before the points: its fraction is of the burst figure of the
    # library's products, and the long batch-64 run before it would put it under the power cap)
    T = 2048
    pre_ms = time_prefill(engine, T)
    flops = prefill_flops(cfg, T)
    prefill = {"value": round(T * 1e3 / pre_ms, 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}

    points = {}
    if point_batches:
        for b in point_batches:
            pms, _, _, _ = time_decode(engine, b, context, max(8, args.steps // 2), args.warmup, 3)
            points[f"decode_b{b}"] = round(b * 1e3 / pms, 1)

    # end to end: the public generate() call, host tokens in and out every step
    # (the steps right after the 8 x 8 000-token prefill run at the clocks that prefill left:
    # 32 of them are let pass before the timed ones)
    e2e_warmup = max(args.warmup, 32)
    n_new = BLOCKS * args.steps + e2e_warmup
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, engine.vocab_size, (context - n_new - 2,), generator=g).tolist()
               for _ in range(batch)]
    stamps = []

    def on_token(index, token):
        if index == 0:
            stamps.append(time.perf_counter())
        return True
    outs = gen.generate(prompts, GenerationConfig(max_tokens=n_new), on_token)
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    timed_tokens = sum(len(o.token_ids) for o in outs) - batch * e2e_warmup
    e2e_value = timed_tokens / (t_end - stamps[e2e_warmup - 1])

    # the other two shapes of the same architecture at full depth, batch 8, same context
    other = {}
    if point_batches and args.shape == "2b" and not args.layers:
        del gen, engine, outs
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for shape in ("9b", "27b"):
            ocfg = baseline_config()
            ocfg.update(SHAPES[shape])
            need = 2 * (ocfg["vocab_size"] * ocfg["hidden_size"] + ocfg["num_hidden_layers"] * (
                ocfg["hidden_size"] * (2 * ocfg["num_attention_heads"]
                                       + 2 * ocfg["num_key_value_heads"]) * ocfg["head_dim"]
                + 3 * ocfg["hidden_size"] * ocfg["intermediate_size"])) \
                + 8 * kv_bytes_per_sequence(ocfg, context)
            if need > 150e9:
                continue
            oeng = GenerationEngine.from_random(ocfg, seed=6 if shape == "9b" else 7,
                                                dtype="bfloat16", ctx=context,
                                                max_tokens=8 * context, max_slots=8).engine
            randomize_pools(oeng)
            oms, olen, _, _ = time_decode(oeng, 8, context, max(8, args.steps // 2), args.warmup, 3)
            obytes = oeng.model.weight_bytes() + kv_bytes_per_step(oeng, olen)
            points[f"decode_b8_{shape}"] = round(8 * 1e3 / oms, 1)
            other[shape] = round(obytes / (oms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
            del oeng
            gc.collect()
            torch.cuda.empty_cache()

    line = {
        "metric": METRIC.replace("2B", args.shape.upper()).replace("batch 8", f"batch {args.batch}")
                  .replace("context 8192", f"context {args.context}"), "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "timed_blocks": BLOCKS, "spread_ms": [round(spread[0], 4), round(spread[1], 4)],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0, 0.02), uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "Gemma2-%s shape" % args.shape.upper(), "global_batch": batch, "seq_len": context,
            "parallelism": "none", "layers": cfg["num_hidden_layers"],
            "layers_of_named_config": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "sliding_window": cfg["sliding_window"],
            "context": context, "kv_len_at_decode": int(statistics.mean(lengths)),
            "l2": "no flush: each step reads more than 5 GB, L2 is 126 MB",
            "peaks": peaks["source"],
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "warmup_steps": e2e_warmup,
                "h2d_bytes_per_step": 8 * batch * 4, "d2h_bytes_per_step": batch * 4,
                "steps_ahead_of_host": 1},
        "gpu_launches": launches * args.steps,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "roofline_other_shapes": other,
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


def run_kernel_tables(args):
    """Where the step's time goes: the decode step of the timed run (same shape, batch and
    context) captured with an event before and after every kernel, and one prompt step."""
    import torch
    from strata_inference_b200 import GenerationEngine
    from strata_inference_b200.engine.profile import (format_table, load_peaks,
                                                      profile_decode_graph, profile_prompt_graph)
    cfg = baseline_config()
    cfg.update(SHAPES[args.shape])
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    context, batch = args.context, args.batch
    gen = GenerationEngine.from_random(cfg, seed=5, dtype="bfloat16", ctx=context,
                                       max_tokens=batch * context, max_slots=batch)
    engine = gen.engine
    randomize_pools(engine)
    peaks = load_peaks()
    slots = [engine.new_sequence() for _ in range(batch)]
    fill_context(engine, slots, context - 16)
    rows, ms = profile_decode_graph(engine, slots, [5] * batch)
    print(format_table(f"Gemma2-{args.shape.upper()} shape, {cfg['num_hidden_layers']} layers: "
                       f"captured decode step, batch {batch}, {context - 16} positions each", rows,
                       ms, peaks))
    for s in slots:
        engine.end_sequence(s)
    T = 2048
    toks = torch.randint(0, engine.vocab_size, (T,), generator=torch.Generator().manual_seed(4)).tolist()
    slot = engine.new_sequence()
    rows, ms = profile_prompt_graph(engine, slot, toks)
    engine.end_sequence(slot)
    print(format_table(f"prompt step, {T} tokens (captured; the events between the kernels keep "
                       f"them from overlapping)", rows, ms, peaks))
    return 0


def run_sweep(args):
    """Decode steps over batch sizes at --context, and prompt steps over lengths: one line
    each with the time, tokens a second and the fraction of the measured peak."""
    import torch
    from strata_inference_b200 import GenerationEngine
    cfg = baseline_config()
    cfg.update(SHAPES[args.shape])
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    context = args.context
    peaks = measured_peaks()
    batches = [b for b in (1, 2, 4, 8, 12, 16, 17, 24, 32, 48, 64, 96, 128)
               if b * kv_bytes_per_sequence(cfg, context) < 120e9]
    top = max(batches)
    gen = GenerationEngine.from_random(cfg, seed=5, dtype="bfloat16", ctx=context,
                                       max_tokens=max(top * context, 2 * 8192), max_slots=top)
    engine = gen.engine
    engine.max_graphs = 2
    randomize_pools(engine)
    weight_bytes = engine.model.weight_bytes()
    print(f"Gemma2-{args.shape.upper()} shape, {cfg['num_hidden_layers']} layers, context {context}: "
          f"decode steps (peak {peaks['hbm_gbs']:.0f} GB/s, {peaks['source']})")
    for b in batches:
        ms, lengths, _, _ = time_decode(engine, b, context, 12, 3, 3)
        moved = weight_bytes + kv_bytes_per_step(engine, lengths)
        print(f"  batch {b:4d}: {ms:7.3f} ms  {b * 1e3 / ms:8.0f} tok/s  "
              f"{moved / (ms * 1e-3) / 1e9 / peaks['hbm_gbs']:.2f} of the copy bandwidth", flush=True)
    print(f"prompt steps, one prompt (peak {peaks['bf16_tflops']:.0f} TFLOP/s)")
    for T in (64, 128, 256, 512, 1024, 2048, 4096, 8192):
        if T > engine.max_seq_len:
            continue
        ms = time_prefill(engine, T, reps=3)
        frac = prefill_flops(cfg, T) / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)
        print(f"  {T:5d} tokens: {ms:7.2f} ms  {T / ms:6.1f} k tok/s  {frac:.2f} of the bf16 peak",
              flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the named configuration (both numbers are reported)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--kernels", action="store_true",
                    help="instead of the timed run: per-kernel tables (CUDA events around every "
                         "kernel) of the captured decode step at --batch and of a 2,048-token "
                         "prompt step, on standard output")
    ap.add_argument("--sweep", action="store_true",
                    help="instead of the timed run: decode steps over batch sizes at --context "
                         "and prompt steps over lengths, one line each, on standard output")
    ap.add_argument("--shape", default="2b", choices=sorted(SHAPES),
                    help="layer sizes: the 2B shape (the recorded line) or the 9B / 27B shapes")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "strata-inference is a Rust crate (Cargo.toml, no setup.py or "
                          "pyproject.toml): pip cannot install it and no Rust toolchain is in "
                          "the image"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this library runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.kernels:
        return run_kernel_tables(args)
    if args.sweep:
        return run_sweep(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
