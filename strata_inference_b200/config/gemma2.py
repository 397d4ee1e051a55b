"""Gemma2: the typed configuration and its translation into a ModelSpec.

Every size and constant comes from ``config.json``; nothing here knows a
model size.  What the architecture fixes (and ``config.json`` has no key
for) is stated once in :func:`gemma2_spec`: tanh-GELU gated feed-forward,
half-split rotary embedding, four ``1 + w`` RMS norms around the two
sub-layers, sqrt(hidden) embedding scale, even layers sliding.

Reference: src/model/config.rs:252-262 (the Gemma defaults: GeGLU, NeoX
rope, embedding scale sqrt(hidden), no biases), :160-229 (optional keys and
their fallbacks), :358-377 (divisibility checks).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, require

_ACTIVATIONS = ("gelu_pytorch_tanh",)
_LAYER_TYPES = ("sliding_attention", "full_attention")


@dataclass(frozen=True)
class Gemma2Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    sliding_window: int            # 0: no layer slides
    query_pre_attn_scalar: float
    attn_logit_softcapping: float  # 0: off
    final_logit_softcapping: float  # 0: off
    rms_norm_eps: float
    max_position_embeddings: int
    hidden_activation: str
    tie_word_embeddings: bool
    layer_types: Tuple[str, ...]
    eos_token_ids: Tuple[int, ...]
    bos_token_id: Optional[int]
    pad_token_id: Optional[int]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Gemma2Config":
        layers = require(d, "num_hidden_layers", int)
        hidden = require(d, "hidden_size", int)
        heads = require(d, "num_attention_heads", int)
        inter = require(d, "intermediate_size", int)
        vocab = require(d, "vocab_size", int)
        theta = float(require(d, "rope_theta", float))
        eps = float(require(d, "rms_norm_eps", float))
        max_pos = require(d, "max_position_embeddings", int)
        for key, v in (("num_hidden_layers", layers), ("hidden_size", hidden),
                       ("num_attention_heads", heads), ("intermediate_size", inter),
                       ("vocab_size", vocab), ("max_position_embeddings", max_pos)):
            if v <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, got {v}")
        if theta <= 0 or eps <= 0:
            raise ConfigError("config.json: 'rope_theta' and 'rms_norm_eps' must be positive")

        kv = d.get("num_key_value_heads")
        kv = heads if kv is None else int(kv)
        if kv <= 0 or heads % kv != 0:
            raise ConfigError(f"config.json: 'num_attention_heads' ({heads}) must be a multiple "
                              f"of 'num_key_value_heads' ({kv})")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(f"config.json: 'hidden_size' ({hidden}) is not a multiple of "
                                  f"'num_attention_heads' ({heads}) and 'head_dim' is not given")
            head_dim = hidden // heads
        head_dim = int(head_dim)
        if head_dim <= 0 or head_dim % 2 != 0:
            raise ConfigError(f"config.json: 'head_dim' must be positive and even, got {head_dim}")

        window = d.get("sliding_window")
        window = 0 if window is None else int(window)
        if window < 0:
            raise ConfigError(f"config.json: 'sliding_window' must be >= 1 or null, got {window}")
        qpas = d.get("query_pre_attn_scalar")
        qpas = float(head_dim) if qpas is None else float(qpas)
        if qpas <= 0:
            raise ConfigError(f"config.json: 'query_pre_attn_scalar' must be positive, got {qpas}")
        attn_cap = float(d.get("attn_logit_softcapping") or 0.0)
        final_cap = float(d.get("final_logit_softcapping") or 0.0)
        if attn_cap < 0 or final_cap < 0:
            raise ConfigError("config.json: soft-capping values must be positive or null")

        act = d.get("hidden_activation") or d.get("hidden_act") or _ACTIVATIONS[0]
        if act not in _ACTIVATIONS:
            raise ConfigError(f"config.json: 'hidden_activation' = {act!r} is not supported; "
                              f"known: {', '.join(_ACTIVATIONS)}")
        if d.get("attention_bias"):
            raise ConfigError("config.json: 'attention_bias' = true is not supported")

        types = d.get("layer_types")
        if types is None:
            types = tuple(_LAYER_TYPES[0] if (i % 2 == 0 and window > 0) else _LAYER_TYPES[1]
                          for i in range(layers))
        else:
            types = tuple(types)
            if len(types) != layers:
                raise ConfigError(f"config.json: 'layer_types' has {len(types)} entries "
                                  f"for {layers} layers")
            for t in types:
                if t not in _LAYER_TYPES:
                    raise ConfigError(f"config.json: 'layer_types' entry {t!r} is not one of "
                                      f"{', '.join(_LAYER_TYPES)}")
            if window == 0 and _LAYER_TYPES[0] in types:
                raise ConfigError("config.json: a sliding layer needs 'sliding_window'")

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        tie = d.get("tie_word_embeddings")
        return cls(
            num_hidden_layers=layers, hidden_size=hidden, num_attention_heads=heads,
            num_key_value_heads=kv, head_dim=head_dim, intermediate_size=inter,
            vocab_size=vocab, rope_theta=theta, sliding_window=window,
            query_pre_attn_scalar=qpas, attn_logit_softcapping=attn_cap,
            final_logit_softcapping=final_cap, rms_norm_eps=eps,
            max_position_embeddings=max_pos, hidden_activation=act,
            tie_word_embeddings=True if tie is None else bool(tie),
            layer_types=types, eos_token_ids=eos_ids,
            bos_token_id=d.get("bos_token_id"), pad_token_id=d.get("pad_token_id"))

    def to_dict(self) -> dict:
        """The config.json of this configuration (random-weights mode writes it)."""
        return {
            "architectures": ["Gemma2ForCausalLM"],
            "model_type": "gemma2",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta,
            "sliding_window": self.sliding_window or None,
            "query_pre_attn_scalar": self.query_pre_attn_scalar,
            "attn_logit_softcapping": self.attn_logit_softcapping or None,
            "final_logit_softcapping": self.final_logit_softcapping or None,
            "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_activation": self.hidden_activation,
            "tie_word_embeddings": self.tie_word_embeddings,
            "layer_types": list(self.layer_types),
            "eos_token_id": list(self.eos_token_ids) if len(self.eos_token_ids) != 1
            else self.eos_token_ids[0],
            "bos_token_id": self.bos_token_id,
            "pad_token_id": self.pad_token_id,
        }


def gemma2_spec(cfg: Gemma2Config) -> ModelSpec:
    """Lay the configuration out as parts, layer by layer."""
    norm = PartSpec("rms_norm", {"eps": cfg.rms_norm_eps, "unit_offset": True})
    rope = PartSpec("rope_neox", {"theta": cfg.rope_theta, "rotary_dim": cfg.head_dim})
    ffn = PartSpec("gated_mlp", {"intermediate_size": cfg.intermediate_size,
                                 "activation": cfg.hidden_activation})
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        mixer = PartSpec("attention", {
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "score_scale": 1.0 / math.sqrt(cfg.query_pre_attn_scalar),
            "logit_softcap": cfg.attn_logit_softcapping,
            "window": cfg.sliding_window if kind == "sliding_attention" else 0,
            "position": rope,
        })
        layers.append(LayerSpec(
            prefix=f"model.layers.{i}.", block="sandwich", mixer=mixer, feed_forward=ffn,
            norms={"pre_mixer": norm, "post_mixer": norm,
                   "pre_feed_forward": norm, "post_feed_forward": norm},
            names={"mixer": "self_attn.", "feed_forward": "mlp.",
                   "pre_mixer": "input_layernorm.",
                   "post_mixer": "post_attention_layernorm.",
                   "pre_feed_forward": "pre_feedforward_layernorm.",
                   "post_feed_forward": "post_feedforward_layernorm."}))
    spec = ModelSpec(
        architecture="Gemma2ForCausalLM",
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"scale": math.sqrt(cfg.hidden_size)}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm,
        head=PartSpec("lm_head", {"tied": cfg.tie_word_embeddings,
                                  "logit_softcap": cfg.final_logit_softcapping}),
        names={"embedding": "model.embed_tokens.", "final_norm": "model.norm.",
               "head": "lm_head."},
        stop_tokens=cfg.eos_token_ids)
    spec.validate()
    return spec
