"""Plain, slow Gemma2: whole sequences, no cache, one function for each part.

This file is the oracle of the test-suite.  It shares no code with the
package: it reads ``config.json`` itself, takes weights as a plain
``{name: torch.Tensor}`` dictionary and recomputes every position of a
sequence from scratch with dense CPU tensor arithmetic.

It rests on the formulas of strata-ai-labs/strata-inference (a Rust crate:
its model code can be neither imported nor compiled where these tests run, so
nothing here was checked against its binaries).  Each function cites the file
and lines of that project that it restates; tests/test_reference_cases.py
applies the inputs and expectations of that project's own unit tests of these
operations to the functions below.  Four formulas are not in that
project's Gemma2 path and are stated here from the architecture's definition
instead: the ``1 + w`` gain of the RMS norms, the ``query_pre_attn_scalar``
score scale, the alternation of sliding and global layers, and the soft cap
on the final logits.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------
# configuration (read directly from config.json's keys)
# --------------------------------------------------------------------------

def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def layer_is_sliding(cfg: dict, i: int) -> bool:
    """Even layers slide, odd layers see everything, unless ``layer_types``
    says otherwise.  (src/model/config.rs:379-385 holds the per-layer flag
    mechanism; it fills it for Gemma3 only.)"""
    types = cfg.get("layer_types")
    if types:
        return types[i] == "sliding_attention"
    return i % 2 == 0 and bool(cfg.get("sliding_window"))


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embed(tokens: Sequence[int], table: torch.Tensor, hidden: int, dtype) -> torch.Tensor:
    """Row gather, then a multiply by sqrt(hidden) taken in f32.
    src/model/layer.rs:1279-1288, src/backend/cpu.rs:1086-1136."""
    idx = torch.as_tensor(list(tokens), dtype=torch.long)
    scale = float(torch.tensor(float(hidden), dtype=torch.float32).sqrt())
    return table.to(dtype)[idx] * scale


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * 1/sqrt(mean(x^2) + eps) * gain with gain = 1 + w.
    src/backend/cpu.rs:797-810 (there the stored weight is the gain)."""
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    inv = 1.0 / torch.sqrt(mean_sq + eps)
    return x * inv * (1.0 + w.to(x.dtype))


def rope_neox(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-split rotary embedding on x[T, heads, head_dim].
    freq_p = theta^((-1/d) * 2p) in f32, angle = pos * freq_p, the pair is
    (x[p], x[p + d/2]).  src/backend/cpu.rs:1276-1322."""
    T, n, d = x.shape
    half = d // 2
    inv_ndims = torch.tensor(-1.0 / d, dtype=torch.float32)
    two_i = torch.arange(half, dtype=torch.float32) * 2.0
    freqs = torch.pow(torch.tensor(theta, dtype=torch.float32), inv_ndims * two_i)
    ang = positions.to(torch.float32)[:, None] * freqs[None, :]
    ang = ang.to(x.dtype)
    cos = torch.cos(ang)[:, None, :]
    sin = torch.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              softcap: float, window: int) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.
    q[T, nh, d], k/v[T, nkv, d].  Scores are scaled, then soft-capped, then
    masked (key j visible to query p iff j <= p and, with a window W,
    p < j + W), then softmax, then the weighted sum of v.
    src/model/layer.rs:1030-1066 (order: scale, cap, mask),
    src/backend/cpu.rs:1352-1434 (grouping, softmax, sum)."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    out = torch.empty_like(q)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible &= pos[:, None] < pos[None, :] + window
    for h in range(nh):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - m)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def gelu_tanh(g: torch.Tensor) -> torch.Tensor:
    """0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))).  src/backend/cpu.rs:1190-1199."""
    c = math.sqrt(2.0 / math.pi)
    return 0.5 * g * (1.0 + torch.tanh(c * (g + 0.044715 * g * g * g)))


def geglu_ffn(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
              w_down: torch.Tensor) -> torch.Tensor:
    """down(gelu_tanh(gate(x)) * up(x)); weights are [out, in], no biases.
    src/model/layer.rs:696-710."""
    return (gelu_tanh(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def attention_block(x: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                    sliding: bool) -> torch.Tensor:
    """q/k/v projections, rotation of q and k, attention, output projection.
    src/model/layer.rs:1113-1161, 906-914."""
    T = x.shape[0]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    d = cfg.get("head_dim", cfg["hidden_size"] // nh)
    q = (x @ W[prefix + "q_proj.weight"].T).view(T, nh, d)
    k = (x @ W[prefix + "k_proj.weight"].T).view(T, nkv, d)
    v = (x @ W[prefix + "v_proj.weight"].T).view(T, nkv, d)
    positions = torch.arange(T)
    theta = float(cfg.get("rope_theta", 10000.0))
    q = rope_neox(q, positions, theta)
    k = rope_neox(k, positions, theta)
    scale = float(cfg.get("query_pre_attn_scalar", d)) ** -0.5
    cap = float(cfg.get("attn_logit_softcapping") or 0.0)
    window = int(cfg.get("sliding_window") or 0) if sliding else 0
    o = attention(q, k, v, scale, cap, window).reshape(T, nh * d)
    return o @ W[prefix + "o_proj.weight"].T


def decoder_layer(h: torch.Tensor, W: Dict[str, torch.Tensor], i: int, cfg: dict) -> torch.Tensor:
    """Pre-norm, mixer, post-norm, add; pre-norm, feed-forward, post-norm, add.
    src/model/layer.rs:1101-1192 (the post norms come before the adds)."""
    p = f"model.layers.{i}."
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    n = rms_norm(h, W[p + "input_layernorm.weight"], eps)
    a = attention_block(n, W, p + "self_attn.", cfg, layer_is_sliding(cfg, i))
    a = rms_norm(a, W[p + "post_attention_layernorm.weight"], eps)
    r = h + a
    n2 = rms_norm(r, W[p + "pre_feedforward_layernorm.weight"], eps)
    f = geglu_ffn(n2, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                  W[p + "mlp.down_proj.weight"])
    f = rms_norm(f, W[p + "post_feedforward_layernorm.weight"], eps)
    return r + f


def lm_head(h: torch.Tensor, W: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """Final norm, product with the output matrix (the embedding table when
    no ``lm_head.weight`` is stored), then cap * tanh(logits / cap).
    src/model/layer.rs:1381-1389, src/engine/generate.rs:1106-1110."""
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    y = rms_norm(h, W["model.norm.weight"], eps)
    out_w = W.get("lm_head.weight", W["model.embed_tokens.weight"])
    logits = y @ out_w.T
    cap = float(cfg.get("final_logit_softcapping") or 0.0)
    if cap > 0:
        logits = cap * torch.tanh(logits / cap)
    return logits


# --------------------------------------------------------------------------
# the whole model
# --------------------------------------------------------------------------

def forward(tokens: Sequence[int], weights: Dict[str, torch.Tensor], cfg: dict,
            dtype=torch.float64) -> torch.Tensor:
    """Logits [T, vocab] of every position of one sequence, from scratch.
    src/model/layer.rs:1255-1392."""
    vocab = cfg["vocab_size"]
    for t in tokens:
        if t >= vocab or t < 0:
            raise ValueError(f"input token ID {t} exceeds vocab_size {vocab}")
    W = {k: v.to(dtype) for k, v in weights.items()}
    h = embed(tokens, W["model.embed_tokens.weight"], cfg["hidden_size"], dtype)
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, W, i, cfg)
    return lm_head(h, W, cfg)


# --------------------------------------------------------------------------
# sampling and generation
# --------------------------------------------------------------------------

class XorShift64:
    """src/engine/sampler.rs:36-58."""

    def __init__(self, seed: int):
        self.state = (seed or 1) & 0xFFFFFFFFFFFFFFFF

    def next_u64(self) -> int:
        x = self.state
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        self.state = x
        return x

    def next_f32(self) -> float:
        return float(self.next_u64() >> 40) / float(1 << 24)


def argmax(logits: Sequence[float]) -> int:
    """First maximum wins.  src/engine/sampler.rs:61-71."""
    best, best_v = 0, float("-inf")
    for i, v in enumerate(logits):
        if v > best_v:
            best, best_v = i, v
    return best


def sample_token(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                 rng: XorShift64) -> int:
    """Temperature, top-k, softmax, top-p, one uniform draw, first index whose
    running sum exceeds it.  src/engine/sampler.rs:82-152."""
    import numpy as np
    l = logits.detach().to(torch.float32).numpy()
    if l.size == 0:
        return 0
    if temperature <= 0.0:
        return int(np.argmax(l))  # numpy's argmax also returns the first maximum
    f32 = np.float32
    cand_idx = np.arange(l.size)
    cand = (l / f32(temperature)).astype(f32)
    if 0 < top_k < l.size:
        order = np.argsort(-cand, kind="stable")[:top_k]
        cand_idx, cand = cand_idx[order], cand[order]
    probs = np.exp(cand - cand.max()).astype(f32)
    probs = (probs / probs.sum(dtype=f32)).astype(f32)
    if top_p < 1.0:
        order = np.argsort(-probs, kind="stable")
        cand_idx, probs = cand_idx[order], probs[order]
        cum = f32(0.0)
        cut = probs.size
        for i, p in enumerate(probs):
            cum = f32(cum + p)
            if cum >= f32(top_p):
                cut = i + 1
                break
        cand_idx, probs = cand_idx[:cut], probs[:cut]
        probs = (probs / probs.sum(dtype=f32)).astype(f32)
    r = f32(rng.next_f32())
    cum = f32(0.0)
    for idx, p in zip(cand_idx, probs):
        cum = f32(cum + p)
        if r < cum:
            return int(idx)
    return int(cand_idx[-1])


def generate(prompt: Sequence[int], weights: Dict[str, torch.Tensor], cfg: dict,
             max_tokens: int, stop_tokens: Sequence[int] = (), temperature: float = 0.0,
             top_k: int = 0, top_p: float = 1.0, seed: Optional[int] = None,
             max_seq_len: Optional[int] = None, dtype=torch.float64):
    """One request, every step recomputed from the first token.
    Order of the decisions: stop token (not emitted), emit, context length,
    next step.  src/engine/generate.rs:655-778."""
    max_seq_len = max_seq_len or cfg.get("max_position_embeddings", 8192)
    if len(prompt) == 0:
        raise ValueError("empty prompt")
    if len(prompt) >= max_seq_len:
        raise ValueError(f"prompt length ({len(prompt)}) exceeds max_seq_len ({max_seq_len})")
    rng = XorShift64(42 if seed is None else seed)
    seq: List[int] = list(prompt)
    out: List[int] = []
    nxt = sample_token(forward(seq, weights, cfg, dtype)[-1], temperature, top_k, top_p, rng)
    reason = "max_tokens"
    for _ in range(max_tokens):
        if nxt in stop_tokens:
            reason = "eos"
            break
        out.append(nxt)
        if len(seq) >= max_seq_len:
            reason = "context_length"
            break
        seq.append(nxt)
        nxt = sample_token(forward(seq, weights, cfg, dtype)[-1], temperature, top_k, top_p, rng)
    return out, reason
