"""Where a step's time goes: CUDA events around every kernel class of one step.

``profile_step(engine, run)`` runs ``run()`` (a prompt step, a single-token step) with
every launcher bracketed by events and returns one row per kernel class with its calls,
device time and the bytes and operations its shapes need; ``format_table`` prints them
with the achieved GB/s or TFLOP/s and the fraction of the device's peak.  The peaks are
the measured copy bandwidth and cuBLAS bfloat16 throughput when a ``MEASURED_PEAKS.json``
lies in the working directory or is named by ``STRATA_PEAKS``, else 6 650 GB/s and
1 590 TFLOP/s (an earlier measurement of a B200).  Launches are not chained while a step
is profiled if ``SIB_CHAINED_LAUNCH=0`` is set; with chaining a kernel's interval may
overlap its predecessor's tail.

The reference prints per-token wall times under ``--profile`` and per-layer times after a
device synchronisation under ``STRATA_PROFILE_LAYERS`` (src/bin/generate.rs:72-74,
src/model/layer.rs:1265,1365-1375).
"""

from __future__ import annotations

import json
import os
from typing import Callable, Dict, List, Tuple

from ..kernels import native


def load_peaks() -> Dict:
    for path in (os.environ.get("STRATA_PEAKS"), "MEASURED_PEAKS.json"):
        if path and os.path.isfile(path):
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def profile_step(run: Callable[[], object]) -> Tuple[List[Dict], float]:
    """(rows, milliseconds of the whole call on the device)."""
    import torch
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with native.KernelProfile() as prof:
        begin.record()
        run()
        end.record()
    rows = prof.rows()
    return rows, begin.elapsed_time(end)


def profile_decode_graph(engine, slots, tokens, replays: int = 3) -> Tuple[List[Dict], float]:
    """The single-token step of ``slots`` as it is served: captured into a CUDA graph with
    an event before and after every kernel, replayed, and read from the last replay.  (The
    event nodes stand between the kernels, so a kernel cannot start under its predecessor's
    tail as it does in the unprofiled graph: the sum is a little above the served step.)
    Advances each sequence by ``replays + 2`` positions."""
    import torch
    from .graph import DecodeGraph
    g = DecodeGraph(engine, len(slots), 0.0, 0, 1.0)
    with native.KernelProfile() as eager:
        g.run(slots, tokens, use_graph=False)
    n = len(eager.events)
    with native.KernelProfile(plan=eager) as captured:
        g.run(slots, tokens, use_graph=True)          # runs once more eagerly, then captures
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(replays):
        if i == replays - 1:
            begin.record()
        g.run(slots, tokens, use_graph=True)
    end.record()
    rows = captured.rows(last=n)
    return rows, begin.elapsed_time(end)


def profile_prompt_graph(engine, slot: int, tokens, replays: int = 3) -> Tuple[List[Dict], float]:
    """A prompt step (``tokens`` for the fresh sequence ``slot``, the last row's logits) with
    an event before and after every kernel, captured into a CUDA graph and replayed, so
    that the host's launch times are not in the figures.  The sequence is advanced once."""
    import torch
    ctx = engine._context([(slot, list(tokens))], None)
    engine.cache.sync_tables()

    def forward():
        h = engine.model.hidden_states(ctx)
        return engine.model.logits(h, ctx.want_rows)
    forward()
    with native.KernelProfile() as eager:
        forward()
    n = len(eager.events)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with native.KernelProfile(plan=eager) as captured:
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            forward()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(replays):
        if i == replays - 1:
            begin.record()
        graph.replay()
    end.record()
    rows = captured.rows(last=n)
    engine.cache.advance(slot, len(tokens))
    return rows, begin.elapsed_time(end)


def format_table(title: str, rows: List[Dict], total_ms: float, peaks: Dict) -> str:
    lines = [f"[profile] {title}: {total_ms * 1e3:.0f} us on the device, "
             f"{sum(r['calls'] for r in rows)} launches; fractions of {peaks['source']} peaks "
             f"({peaks['hbm_gbs']:.0f} GB/s, {peaks['bf16_tflops']:.0f} TFLOP/s)",
             f"[profile] {'kernel':<40} {'calls':>5} {'us':>9} {'us/call':>8} {'GB/s':>8} "
             f"{'TFLOP/s':>8} {'of peak':>7}"]
    for r in rows:
        s = r["ms"] * 1e-3
        gbs = r["bytes"] / s / 1e9 if s > 0 else 0.0
        tf = r["flops"] / s / 1e12 if s > 0 else 0.0
        frac = max(gbs / peaks["hbm_gbs"], tf / peaks["bf16_tflops"])
        lines.append(f"[profile] {r['name']:<40} {r['calls']:>5} {r['ms'] * 1e3:>9.1f} "
                     f"{r['ms'] * 1e3 / r['calls']:>8.1f} {gbs:>8.0f} {tf:>8.1f} {frac:>7.2f}")
    inside = sum(r["ms"] for r in rows)
    lines.append(f"[profile] {'(between kernels)':<40} {'':>5} {(total_ms - inside) * 1e3:>9.1f}")
    return "\n".join(lines)
