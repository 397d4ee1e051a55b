"""Shared by the tests: the tiny configurations, model folders in temporary
directories, and the comparison against the plain implementation."""

from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import torch

import plain_gemma2 as plain

# Tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "vocab_size": 256,
    "rope_theta": 10000.0, "sliding_window": 8, "query_pre_attn_scalar": 16,
    "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 128, "hidden_activation": "gelu_pytorch_tanh",
    "tie_word_embeddings": True, "eos_token_id": 1,
}
TINY_B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 320, "vocab_size": 512,
    "rope_theta": 500000.0, "sliding_window": 16, "query_pre_attn_scalar": 24,
    "attn_logit_softcapping": None, "final_logit_softcapping": None, "rms_norm_eps": 1e-5,
    "max_position_embeddings": 64, "hidden_activation": "gelu_pytorch_tanh",
    "tie_word_embeddings": True, "eos_token_id": [1, 7],
}
# One kv head, a head size that is a multiple of 16 but not of 32, a vocabulary
# that is no multiple of 16, layer kinds given explicitly, untied head.
TINY_C = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 4, "hidden_size": 80, "num_attention_heads": 5,
    "num_key_value_heads": 1, "head_dim": 48, "intermediate_size": 200, "vocab_size": 300,
    "rope_theta": 2500.0, "sliding_window": 24, "query_pre_attn_scalar": 30,
    "attn_logit_softcapping": 20.0, "final_logit_softcapping": None, "rms_norm_eps": 1e-4,
    "max_position_embeddings": 256, "hidden_activation": "gelu_pytorch_tanh",
    "tie_word_embeddings": False,
    "layer_types": ["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}

# Largest allowed |engine - plain| as a fraction of the largest |plain| logit of
# the compared rows.  32-bit: a few rounding errors of 2^-24 through a handful of
# layers.  bfloat16: activations are rounded to 8 bits of mantissa (2^-9 relative)
# between kernels, and a few tens of such roundings add up along a layer stack.
REL_TOL = {"float32": 2e-5, "bfloat16": 3e-2}

# How much the q and k projections of the test models are scaled up.  Sharp
# attention makes a wrong key, mask edge or cache cell visible, which the 32-bit
# runs check to 2e-5.  In bfloat16 the rounding of q and k (2^-9 relative) shifts
# each score by about that fraction of its size, and the softmax turns the shift
# into a relative error of the weights: measured on these configurations, the
# largest logit error grows from 0.6-0.9 % of the largest logit at factor 1 to
# 1.6-5 % at factor 2.  The bfloat16 runs therefore use factor 1, where rounding
# stays well below the tolerance and anything above it is a fault.
SHARPEN = {"float32": 2.0, "bfloat16": 1.0}


def make_model_dir(path: str, cfg: dict, seed: int, store: torch.dtype = torch.bfloat16,
                   sharpen: float = 2.0) -> str:
    """A model folder with seeded random weights.  q and k projections are
    scaled up by ``sharpen`` so that attention is far from uniform and a wrong
    key, mask edge or cache cell changes the logits visibly."""
    from strata_inference_b200.weights.random_init import write_random_model
    from strata_inference_b200.weights.safetensors_io import ModelFiles, write_safetensors
    write_random_model(path, cfg, seed, torch.float32, matrix_std=0.08, norm_std=0.3)
    files = ModelFiles(path)
    tensors = {}
    for n in files.names():
        t = files.get(n).clone()
        if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
            t = t * sharpen
        tensors[n] = t.to(store)
    write_safetensors(os.path.join(path, "model.safetensors"), tensors)
    return path


def plain_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    """The stored tensors, read with the safetensors package (not with the
    library under test)."""
    from safetensors.torch import load_file
    return load_file(os.path.join(model_dir, "model.safetensors"))


def eos_list(cfg: dict) -> List[int]:
    """The stop tokens that config.json names."""
    eos = cfg.get("eos_token_id")
    if eos is None:
        return []
    return list(eos) if isinstance(eos, (list, tuple)) else [eos]


def random_prompts(cfg: dict, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]


def plain_logits(tokens: Sequence[int], model_dir: str, cfg: dict) -> torch.Tensor:
    return plain.forward(tokens, plain_weights(model_dir), cfg, dtype=torch.float64)


def assert_logits_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "") -> None:
    got = got.detach().to("cpu", torch.float64)
    ref = ref.to(torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = ref.abs().max().item()
    err = (got - ref).abs().max().item()
    assert err <= REL_TOL[dtype] * scale, (
        f"{what}: max |diff| {err:.3e} exceeds {REL_TOL[dtype]:.0e} x max|ref| {scale:.3e} "
        f"(first bad row {int(((got - ref).abs().amax(dim=-1) > REL_TOL[dtype] * scale).nonzero()[0])})")


def assert_greedy_choices_close(prompt: Sequence[int], tokens: Sequence[int], weights, cfg: dict,
                                dtype: str, what: str = "") -> None:
    """Greedy tokens of a reduced-precision run cannot be compared token for token with the
    plain implementation's (one near-tie sends the two apart), but each choice can: given
    the run's own history, the chosen token's plain logit must lie within rounding of the
    plain maximum at that position.  A wrong but stable token fails this."""
    logits = plain.forward(list(prompt) + list(tokens), weights, cfg, dtype=torch.float64)
    for k, tok in enumerate(tokens):
        row = logits[len(prompt) + k - 1]
        gap = (row.max() - row[tok]).item()
        assert gap <= 2 * REL_TOL[dtype] * row.abs().max().item(), (
            f"{what}: token {k} ({tok}) lies {gap:.3e} below the best logit "
            f"({int(row.argmax())}, {row.max().item():.3e})")
