"""Configuration and registry (no device needed)."""

import json
import math

import pytest

from helpers import CONFIGS, TINY_A, TINY_B, TINY_C
from strata_inference_b200.config.gemma2 import Gemma2Config, gemma2_spec
from strata_inference_b200.config.registry import (architecture_of, known_architectures,
                                                   read_config_json, spec_from_config)
from strata_inference_b200.config.spec import ConfigError, ModelSpec, PartSpec, ScheduleEntry


def test_every_size_comes_from_config_json():
    for cfg in CONFIGS.values():
        typed, spec = spec_from_config(cfg)
        assert isinstance(typed, Gemma2Config)
        assert spec.hidden_size == cfg["hidden_size"] and spec.vocab_size == cfg["vocab_size"]
        assert spec.max_positions == cfg["max_position_embeddings"]
        assert len(spec.layers) == cfg["num_hidden_layers"]
        assert spec.embedding.params["scale"] == math.sqrt(cfg["hidden_size"])
        assert spec.head.params["logit_softcap"] == (cfg["final_logit_softcapping"] or 0.0)
        assert spec.head.params["tied"] == cfg["tie_word_embeddings"]
        for layer in spec.layers:
            m = layer.mixer.params
            assert m["num_heads"] == cfg["num_attention_heads"]
            assert m["num_kv_heads"] == cfg["num_key_value_heads"]
            assert m["head_dim"] == cfg["head_dim"]
            assert m["score_scale"] == pytest.approx(cfg["query_pre_attn_scalar"] ** -0.5, rel=1e-15)
            assert m["logit_softcap"] == (cfg["attn_logit_softcapping"] or 0.0)
            assert m["position"].params["theta"] == cfg["rope_theta"]
            assert layer.feed_forward.params["intermediate_size"] == cfg["intermediate_size"]
            for norm in layer.norms.values():
                assert norm.params["eps"] == cfg["rms_norm_eps"] and norm.params["unit_offset"]


def test_layers_alternate_unless_layer_types_says_otherwise():
    _, a = spec_from_config(TINY_A)
    assert [l.mixer.params["window"] for l in a.layers] == [8, 0]
    _, b = spec_from_config(TINY_B)
    assert [l.mixer.params["window"] for l in b.layers] == [16, 0, 16]
    _, c = spec_from_config(TINY_C)
    assert [l.mixer.params["window"] for l in c.layers] == [0, 24, 24, 0]
    no_window = dict(TINY_A, sliding_window=None)
    _, n = spec_from_config(no_window)
    assert [l.mixer.params["window"] for l in n.layers] == [0, 0]


def test_defaults_that_are_derived():
    cfg = {k: v for k, v in TINY_A.items()
           if k not in ("num_key_value_heads", "head_dim", "query_pre_attn_scalar")}
    typed, _ = spec_from_config(cfg)
    assert typed.num_key_value_heads == 4 and typed.head_dim == 16
    assert typed.query_pre_attn_scalar == 16.0
    assert typed.eos_token_ids == (1,)
    assert spec_from_config(TINY_B)[0].eos_token_ids == (1, 7)


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads",
                                 "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps",
                                 "max_position_embeddings"])
def test_missing_key_is_named(key):
    cfg = {k: v for k, v in TINY_A.items() if k != key}
    with pytest.raises(ConfigError, match=key):
        spec_from_config(cfg)


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 15}, "head_dim"),
    ({"hidden_activation": "relu"}, "hidden_activation"),
    ({"sliding_window": -1}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["full_attention", "chunked"]}, "chunked"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"num_hidden_layers": "2"}, "num_hidden_layers"),
    ({"attention_bias": True}, "attention_bias"),
    ({"query_pre_attn_scalar": 0}, "query_pre_attn_scalar"),
])
def test_invalid_values_are_refused(change, match):
    with pytest.raises(ConfigError, match=match):
        spec_from_config(dict(TINY_A, **change))


def test_unknown_architecture_lists_the_known_ones():
    with pytest.raises(ConfigError) as e:
        architecture_of({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    assert "LlamaForCausalLM" in str(e.value) and "Gemma2ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        architecture_of({})
    assert "gemma2" in known_architectures()
    assert architecture_of({"model_type": "gemma2"}).name == "Gemma2ForCausalLM"


def test_config_round_trip(tmp_path):
    typed, _ = spec_from_config(TINY_C)
    (tmp_path / "config.json").write_text(json.dumps(typed.to_dict()))
    again, _ = spec_from_config(read_config_json(str(tmp_path)))
    assert again == typed
    with pytest.raises(ConfigError, match="no such file"):
        read_config_json(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))


def test_schedule_is_data_and_is_checked():
    _, spec = spec_from_config(TINY_A)
    ok = ModelSpec(**{**spec.__dict__, "schedule": (ScheduleEntry(0), ScheduleEntry(1),
                                                    ScheduleEntry(0), ScheduleEntry(1, cache_of=1))})
    ok.validate()
    for bad in [(ScheduleEntry(2),), (ScheduleEntry(0, cache_of=0),),
                (ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(0, cache_of=1))]:
        with pytest.raises(ConfigError):
            ModelSpec(**{**spec.__dict__, "schedule": bad}).validate()


def test_unknown_part_kind_is_an_error_that_lists_kinds():
    from strata_inference_b200.engine.model import expected_tensors
    _, spec = spec_from_config(TINY_A)
    layers = list(spec.layers)
    l0 = layers[0]
    layers[0] = type(l0)(**{**l0.__dict__, "mixer": PartSpec("no_such_mixer", {})})
    broken = ModelSpec(**{**spec.__dict__, "layers": tuple(layers)})
    with pytest.raises(ConfigError, match="no_such_mixer.*attention|attention.*no_such_mixer"):
        expected_tensors(broken)
