"""Command line, in the manner of the reference's ``strata-generate``
(src/bin/generate.rs:19-84): the same option names with the same meanings
and defaults where the reference has them.

    python -m strata_inference_b200.cli -m MODEL_DIR --token-ids 2,17,5 -n 16 --temp 0

Differences that follow from what this library is: ``-m`` names a folder
with config.json and safetensors; there is no tokenizer, so ``-p`` and
``-f`` take token ids (separated by commas or blanks; in a file, one request
per line) and ``--token-ids`` may be repeated, one request each; the
requests run as one batch.  ``--backend`` accepts ``auto`` and ``cuda``.
Added: ``--dtype``, ``--cache-tokens``, ``--stop-token``, and
``--random-weights SEED`` which first writes MODEL_DIR (a config.json must
be there or be given with ``--config``).  ``--dump-logits FILE`` writes the
32-bit logits each generated token was chosen from, one comma-separated line
per token (single request only); the reference declares this option but
writes token ids (src/bin/generate.rs:236-251).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional


def _ids(text: str) -> List[int]:
    parts = text.replace(",", " ").split()
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"Error: invalid token ID in {text!r}")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="strata-generate",
                                 description="Generate token ids from a model folder")
    ap.add_argument("-m", "--model", required=True, help="folder with config.json and safetensors")
    ap.add_argument("-p", "--prompt", help="prompt as token ids")
    ap.add_argument("-f", "--file", help="read prompts (token ids, one request per line) from a file")
    ap.add_argument("--token-ids", action="append",
                    help="comma-separated token ids; repeat for several requests")
    ap.add_argument("-n", "--max-tokens", type=int, default=-1,
                    help="maximum tokens to generate (-1 = until a stop token or the context limit)")
    ap.add_argument("--temp", type=float, default=0.8, help="temperature (0.0 = greedy)")
    ap.add_argument("--top-k", type=int, default=40, help="top-k sampling (0 = disabled)")
    ap.add_argument("--top-p", type=float, default=0.95, help="top-p (nucleus) sampling")
    ap.add_argument("-s", "--seed", type=int, default=None, help="random seed for sampling")
    ap.add_argument("--no-display-prompt", action="store_true", help="don't echo the prompt")
    ap.add_argument("--output-format", choices=["text", "json"], default="text")
    ap.add_argument("--backend", default="auto", help="compute backend: auto, cuda")
    ap.add_argument("--log-disable", action="store_true", help="suppress all logging")
    ap.add_argument("--profile", action="store_true",
                    help="per-token times, and per-kernel times of one prompt step and one "
                         "single-token step, on standard error (also: STRATA_PROFILE=1)")
    ap.add_argument("-c", "--ctx", type=int, default=None,
                    help="context length override (lowers the maximum sequence length)")
    ap.add_argument("--dump-logits", default=None,
                    help="write the logits of each generated token to a file")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--cache-tokens", type=int, default=None,
                    help="positions the cache holds (default: enough for the requests)")
    ap.add_argument("--stop-token", type=int, action="append", default=[],
                    help="stop when this token is produced (repeatable)")
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="write seeded random weights into the model folder first")
    ap.add_argument("--config", default=None, help="config.json to use with --random-weights")
    return ap


def _print_kernel_tables(engine, prompt: List[int]) -> None:
    """The first request's prompt as one step and one single-token step after it, run once
    more with CUDA events around every kernel."""
    from .engine.profile import (format_table, load_peaks, profile_decode_graph,
                                 profile_prompt_graph)
    peaks = load_peaks()
    slot = engine.new_sequence()
    try:
        rows, ms = profile_prompt_graph(engine, slot, prompt)
        print(format_table(f"prompt step, {len(prompt)} tokens (captured, events between the "
                           f"kernels)", rows, ms, peaks), file=sys.stderr)
        if engine.length(slot) + 5 < engine.max_seq_len:
            rows, ms = profile_decode_graph(engine, [slot], [prompt[-1]])
            print(format_table(f"single-token step near position {engine.length(slot)} "
                               f"(captured, events between the kernels)", rows, ms, peaks),
                  file=sys.stderr)
    finally:
        engine.end_sequence(slot)


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if os.environ.get("STRATA_PROFILE", "") not in ("", "0"):
        args.profile = True
    given = [x is not None for x in (args.prompt, args.file, args.token_ids)]
    if sum(given) != 1:
        print("Error: give exactly one of --prompt, --file, --token-ids", file=sys.stderr)
        return 1
    if args.backend not in ("auto", "cuda"):
        print(f"Error: unknown backend '{args.backend}'. Options: auto, cuda", file=sys.stderr)
        return 1
    if args.prompt is not None:
        prompts = [_ids(args.prompt)]
    elif args.file is not None:
        with open(args.file) as f:
            prompts = [_ids(line) for line in f if line.strip()]
    else:
        prompts = [_ids(t) for t in args.token_ids]

    def log(msg: str) -> None:
        if not args.log_disable:
            print(msg, file=sys.stderr, flush=True)

    try:
        import torch
        from . import GenerationConfig, GenerationEngine, SamplingConfig, write_random_model
        total_start = time.perf_counter()
        if args.random_weights is not None:
            cfg_path = args.config or os.path.join(args.model, "config.json")
            with open(cfg_path) as f:
                config = json.load(f)
            write_random_model(args.model, config, args.random_weights, torch.bfloat16,
                               device="cuda:0" if torch.cuda.is_available() else "cpu")
            log(f"wrote random weights (seed {args.random_weights}) to {args.model}")
        need = args.cache_tokens
        if need is None:
            per = 8192 if args.max_tokens < 0 else max(len(p) for p in prompts) + args.max_tokens
            need = len(prompts) * (-(-per // 64) * 64)
        load_start = time.perf_counter()
        engine = GenerationEngine.from_dir(args.model, dtype=args.dtype, ctx=args.ctx,
                                           max_tokens=need)
        load_ms = (time.perf_counter() - load_start) * 1e3
        # (the logits of every token are dumped from inside the token callback: the device
        # must then not be a step ahead of it)
        conf = GenerationConfig(
            max_tokens=args.max_tokens, stop_tokens=args.stop_token,
            sampling=SamplingConfig(temperature=args.temp, top_k=args.top_k, top_p=args.top_p,
                                    seed=args.seed),
            look_ahead=not args.dump_logits)
        first_token_at = [None]
        last = [time.perf_counter()]
        dump = open(args.dump_logits, "w") if args.dump_logits and len(prompts) == 1 else None
        if args.dump_logits and dump is None:
            log("--dump-logits takes a single request; ignored")

        def on_token(index: int, token: int) -> bool:
            now = time.perf_counter()
            if first_token_at[0] is None:
                first_token_at[0] = now
            if args.profile:
                print(f"[profile] request {index} token {token}: {(now - last[0]) * 1e3:.2f}ms",
                      file=sys.stderr)
            last[0] = now
            if dump is not None:
                row = engine.last_logits()
                if row is not None:
                    dump.write(",".join(repr(float(v)) for v in row[0].tolist()) + "\n")
            return True

        gen_start = time.perf_counter()
        outs = engine.generate(prompts, conf, on_token)
        end = time.perf_counter()
        if dump is not None:
            dump.close()
        if args.profile:
            _print_kernel_tables(engine.engine, prompts[0])
    except Exception as e:  # one line, as the reference prints it
        print(f"Error: {e}", file=sys.stderr)
        return 1

    prefill_s = max(o.prefill_duration for o in outs)
    decode_s = end - (first_token_at[0] or end)
    n_prompt = sum(o.prompt_tokens for o in outs)
    n_gen = sum(len(o.token_ids) for o in outs)
    timings = {
        "load_ms": load_ms, "prefill_ms": prefill_s * 1e3, "decode_ms": decode_s * 1e3,
        "total_ms": (end - total_start) * 1e3,
        "prefill_tok_per_sec": n_prompt / prefill_s if prefill_s > 0 else 0.0,
        "decode_tok_per_sec": n_gen / decode_s if decode_s > 0 else 0.0,
    }
    conf_out = {"max_tokens": args.max_tokens, "temperature": args.temp, "top_k": args.top_k,
                "top_p": args.top_p, "seed": args.seed}
    records = []
    for p, o in zip(prompts, outs):
        records.append({
            "model": args.model, "prompt": f"[{len(p)} token IDs]",
            "output": " ".join(map(str, o.token_ids)), "output_token_ids": o.token_ids,
            "generated_tokens": len(o.token_ids), "stop_reason": o.stop_reason,
            "timings": timings, "config": conf_out})
    if args.output_format == "json":
        print(json.dumps(records[0] if len(records) == 1 else records, indent=2))
    else:
        for p, o in zip(prompts, outs):
            if not args.no_display_prompt:
                print(" ".join(map(str, p)), end=" | ")
            print(" ".join(map(str, o.token_ids)))
        log(f"{n_gen} tokens, {o.stop_reason}; prefill {timings['prefill_tok_per_sec']:.1f} tok/s, "
            f"decode {timings['decode_tok_per_sec']:.1f} tok/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
