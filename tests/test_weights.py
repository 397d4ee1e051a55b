"""Safetensors reading and writing, checked loading and its one error, and the
random-weights mode (no device needed)."""

import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, TINY_C
from strata_inference_b200.config.registry import spec_from_config
from strata_inference_b200.engine.model import expected_tensors
from strata_inference_b200.weights.loader import (TensorDecl, WeightError, check_table,
                                                  load_weights, storage_dtype)
from strata_inference_b200.weights.random_init import random_tensors, write_random_model
from strata_inference_b200.weights.safetensors_io import (ModelFiles, SafetensorsError,
                                                          SafetensorsFile, write_safetensors)


def test_round_trip_against_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    g = torch.Generator().manual_seed(0)
    tensors = {"a.weight": torch.randn(3, 5, generator=g),
               "b": torch.randn(7, generator=g).to(torch.bfloat16),
               "c.table": torch.arange(6, dtype=torch.int64).view(2, 3),
               "d": torch.randn(2, 2, generator=g).to(torch.float16)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, {"format": "pt"})
    theirs = load_file(path)
    ours = SafetensorsFile(path)
    assert set(ours.names()) == set(tensors)
    for n, t in tensors.items():
        assert torch.equal(theirs[n], t) and torch.equal(ours.get(n), t)
        assert ours.shape(n) == tuple(t.shape) and ours.dtype(n) == t.dtype
    save_file(tensors, str(tmp_path / "y.safetensors"))
    assert torch.equal(SafetensorsFile(str(tmp_path / "y.safetensors")).get("b"), tensors["b"])


def test_sharded_folder(tmp_path):
    write_safetensors(str(tmp_path / "model-00001.safetensors"), {"a": torch.ones(2)})
    write_safetensors(str(tmp_path / "model-00002.safetensors"), {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "model-00001.safetensors", "b": "model-00002.safetensors"}}))
    files = ModelFiles(str(tmp_path))
    assert sorted(files.names()) == ["a", "b"] and files.get("b").shape == (3,)


def test_broken_files_are_refused(tmp_path):
    with pytest.raises(SafetensorsError, match="neither"):
        ModelFiles(str(tmp_path))
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        ModelFiles(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        ModelFiles(str(tmp_path))
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="'w'"):
        ModelFiles(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    _, spec = spec_from_config(TINY_A)
    expected = expected_tensors(spec)
    tensors = random_tensors(expected, 0, torch.bfloat16)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63, dtype=torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16)
    tensors["lm_head.weight"] = torch.zeros(256, 64)        # tied: nobody asks for it
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        load_weights(str(tmp_path), expected, torch.device("cpu"))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["lm_head.weight", "model.layers.0.self_attn.q_norm.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 63), (64, 64))]
    assert [n for n, _ in err.wrong_kind] == ["model.layers.0.input_layernorm.weight"]
    text = str(err)
    for piece in ("missing (2)", "unexpected (2)", "wrong shape (1)", "[64, 63]", "[64, 64]",
                  "model.norm.weight", "q_norm"):
        assert piece in text


def test_expected_tensors_of_the_three_configs():
    for cfg in (TINY_A, TINY_B, TINY_C):
        _, spec = spec_from_config(cfg)
        exp = expected_tensors(spec)
        L, H, I = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"]
        nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        assert len(exp) == 2 + 11 * L + (0 if cfg["tie_word_embeddings"] else 1)
        assert exp["model.embed_tokens.weight"].shape == (cfg["vocab_size"], H)
        assert exp["model.layers.0.self_attn.q_proj.weight"].shape == (nh * hd, H)
        assert exp[f"model.layers.{L - 1}.self_attn.v_proj.weight"].shape == (nkv * hd, H)
        assert exp["model.layers.0.self_attn.o_proj.weight"].shape == (H, nh * hd)
        assert exp["model.layers.0.mlp.down_proj.weight"].shape == (H, I)
        assert exp["model.layers.0.post_feedforward_layernorm.weight"] == TensorDecl((H,), "norm")
        assert ("lm_head.weight" in exp) == (not cfg["tie_word_embeddings"])


def test_stored_types_are_kept():
    assert storage_dtype(torch.bfloat16) == torch.bfloat16
    assert storage_dtype(torch.float32) == torch.float32
    assert storage_dtype(torch.float16) == torch.bfloat16
    assert storage_dtype(torch.int64) == torch.int32


def test_loading_keeps_32_bit_tensors_and_bfloat16(tmp_path):
    _, spec = spec_from_config(TINY_A)
    expected = expected_tensors(spec)
    tensors = random_tensors(expected, 1, torch.bfloat16)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() + 1e-4   # not bf16-exact
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    loaded = load_weights(str(tmp_path), expected, torch.device("cpu"))
    assert loaded["model.norm.weight"].dtype == torch.float32
    assert torch.equal(loaded["model.norm.weight"], tensors["model.norm.weight"])
    assert loaded["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_random_weights_mode_writes_a_loadable_reproducible_folder(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_B, seed=2)
    b = write_random_model(str(tmp_path / "b"), TINY_B, seed=2)
    c = write_random_model(str(tmp_path / "c"), TINY_B, seed=3)
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(a, "config.json"))) == TINY_B
    fa, fb, fc = ModelFiles(a), ModelFiles(b), ModelFiles(c)
    _, spec = spec_from_config(TINY_B)
    check_table(a, {n: (fa.shape(n), fa.dtype(n)) for n in fa.names()}, expected_tensors(spec))
    for n in fa.names():
        assert torch.equal(fa.get(n), fb.get(n))
    assert not torch.equal(fa.get("model.embed_tokens.weight"), fc.get("model.embed_tokens.weight"))
    emb = fa.get("model.embed_tokens.weight").float()
    norm = torch.cat([fa.get(n).float() for n in fa.names() if "norm" in n])
    assert abs(emb.std().item() - 0.02) < 0.002 and abs(norm.std().item() - 0.1) < 0.02
    assert fa.dtype("model.embed_tokens.weight") == torch.bfloat16
    # a tensor's values do not depend on which other tensors exist
    _, spec_a = spec_from_config(dict(TINY_B, num_hidden_layers=1))
    fewer = random_tensors(expected_tensors(spec_a), 2, torch.bfloat16)
    assert torch.equal(fewer["model.layers.0.mlp.up_proj.weight"],
                       fa.get("model.layers.0.mlp.up_proj.weight"))
