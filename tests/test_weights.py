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
    tensors["lm_head.weight"] = torch.zeros(256, 64)        # tied: accepted and not read
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        load_weights(str(tmp_path), expected, torch.device("cpu"))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 63), (64, 64))]
    assert [n for n, _ in err.wrong_kind] == ["model.layers.0.input_layernorm.weight"]
    text = str(err)
    for piece in ("missing (2)", "unexpected (1)", "wrong shape (1)", "[64, 63]", "[64, 64]",
                  "model.norm.weight", "q_norm"):
        assert piece in text


def test_expected_tensors_of_the_three_configs():
    for cfg in (TINY_A, TINY_B, TINY_C):
        _, spec = spec_from_config(cfg)
        exp = expected_tensors(spec)
        L, H, I = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"]
        nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        assert len(exp) == 3 + 11 * L
        assert exp["lm_head.weight"].optional == bool(cfg["tie_word_embeddings"])
        assert exp["model.embed_tokens.weight"].shape == (cfg["vocab_size"], H)
        assert exp["model.layers.0.self_attn.q_proj.weight"].shape == (nh * hd, H)
        assert exp[f"model.layers.{L - 1}.self_attn.v_proj.weight"].shape == (nkv * hd, H)
        assert exp["model.layers.0.self_attn.o_proj.weight"].shape == (H, nh * hd)
        assert exp["model.layers.0.mlp.down_proj.weight"].shape == (H, I)
        assert exp["model.layers.0.post_feedforward_layernorm.weight"] == TensorDecl((H,), "norm")


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


# ---------------------------------------------------------------- the seeded generator

def _restated_normal(key: int, i: int) -> float:
    """Element i of the tensor with `key`, one scalar at a time with numpy's 32-bit
    scalars: the formula of weights/random_init.py and csrc/randn_fill.cu written out
    again, sharing nothing with either."""
    import numpy as np
    f = np.float32
    M = (1 << 64) - 1

    def mix(z):
        z ^= z >> 30
        z = (z * 0xBF58476D1CE4E5B9) & M
        z ^= z >> 27
        z = (z * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)
    h = mix((key + (i + 1) * 0x9E3779B97F4A7C15) & M)
    u1 = f((h >> 40) + 1) * f(2.0 ** -24)
    a = (h >> 8) & 0xFFFFFF
    quadrant, t = a >> 22, f(a & 0x3FFFFF) * f(2.0 ** -22)
    # ln u1
    bits = int(np.array(u1, dtype=np.float32).view(np.int32))
    e = (bits >> 23) - 127
    m = np.array((bits & 0x007FFFFF) | 0x3F800000, dtype=np.int32).view(np.float32)[()]
    if m > f(1.41421354):
        m, e = m * f(0.5), e + 1
    s = (m + f(-1.0)) / (m + f(1.0))
    s2 = s * s
    p = f(0.111111111)
    for c in (0.142857143, 0.2, 0.333333333, 1.0):
        p = p * s2 + f(c)
    ln = f(e) * f(0.693147181) + (f(2.0) * s) * p
    # cos(2 pi a / 2^24) by quadrants
    if quadrant in (1, 3):
        t = f(1.0) + (-t)
    x = t * f(1.57079633)
    x2 = x * x
    p = f(-1.14707456e-11)
    for c in (2.08767570e-9, -2.75573192e-7, 2.48015873e-5, -1.38888889e-3, 4.16666667e-2,
              -0.5, 1.0):
        p = p * x2 + f(c)
    if quadrant in (1, 2):
        p = -p
    return float(np.sqrt(f(-2.0) * ln) * p)


def test_generator_is_one_formula_of_seed_name_and_index():
    import numpy as np
    from strata_inference_b200.weights.random_init import randn_host, tensor_key
    name, seed, std = "model.layers.3.mlp.up_proj.weight", 5, 0.02
    got = randn_host((7, 33), seed, name, std)
    key = tensor_key(seed, name)
    with np.errstate(over="ignore"):
        want = [float(np.float32(std) * np.float32(_restated_normal(key, i))) for i in range(7 * 33)]
    assert got.flatten().tolist() == want                      # to the bit
    # the key: FNV-1a of the name mixed with the seed, nothing else
    assert tensor_key(5, name) != tensor_key(6, name) != tensor_key(5, name + "x")
    # and what comes out is a standard normal
    z = randn_host((1 << 20,), 9, "t", 1.0).double()
    assert abs(z.mean().item()) < 4e-3 and abs(z.std().item() - 1.0) < 4e-3
    assert abs((z ** 3).mean().item()) < 2e-2 and abs((z ** 4).mean().item() - 3.0) < 5e-2
    assert 4.5 < z.abs().max().item() < 6.0
    # cos and ln as evaluated are within 32-bit rounding of the functions
    import math
    for i in range(0, 4000, 7):
        a = (i * 4099) & 0xFFFFFF
        h = (a << 8) | (((i * 2654435761) & 0xFFFFFF) << 40)
        # (a hash with these bits would give this angle and this u1)
        u1 = ((h >> 40) + 1) * 2.0 ** -24
        exact = math.sqrt(-2.0 * math.log(u1)) * math.cos(2.0 * math.pi * a / 2 ** 24)
        import strata_inference_b200.weights.random_init as ri
        with np.errstate(over="ignore"):
            t = (np.array([a & 0x3FFFFF], dtype=np.uint32)).astype(np.float32) * np.float32(2.0 ** -22)
            q = a >> 22
            c = ri._cos_quarter(np.float32(1.0) + (-t) if q in (1, 3) else t)
            c = -c if q in (1, 2) else c
            r = np.sqrt(np.float32(-2.0) * ri._ln_unit(np.array([u1], dtype=np.float32)))
        assert abs(float((r * c)[0]) - exact) < 3e-6 * max(1.0, abs(exact))


def test_arena_places_stored_tensors_without_a_second_copy():
    """The resident tensors of a model (q|k|v as one matrix, gate and up interleaved, the
    norms' 1 + w) are views of ONE buffer, and each source fills them alike."""
    from strata_inference_b200.engine.model import place_weights, resident_plan
    from strata_inference_b200.weights.arena import DictSource, RandomSource
    cfg = TINY_B
    _, spec = spec_from_config(cfg)
    expected = expected_tensors(spec)
    stored = random_tensors(expected, 4, torch.bfloat16)
    arena = place_weights(spec, DictSource(stored), torch.float32, "cpu")
    plan = resident_plan(spec)
    assert set(arena.tensors) == set(plan)
    base = arena.buffer.data_ptr()
    for t in arena.tensors.values():
        assert 0 <= t.data_ptr() - base < arena.buffer.numel() and (t.data_ptr() - base) % 256 == 0
    p = "model.layers.1."
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qkv = arena.tensors[p + "self_attn.qkv_proj.weight"]
    assert qkv.dtype == torch.float32 and qkv.shape == ((nh + 2 * nkv) * hd, cfg["hidden_size"])
    want = torch.cat([stored[p + f"self_attn.{n}_proj.weight"] for n in "qkv"]).float()
    assert torch.equal(qkv, want)
    I, H = cfg["intermediate_size"], cfg["hidden_size"]
    gu = arena.tensors[p + "mlp.gate_up_proj.weight"].view(I // 8, 2, 8, H)
    assert torch.equal(gu[:, 0].reshape(I, H), stored[p + "mlp.gate_proj.weight"].float())
    assert torch.equal(gu[:, 1].reshape(I, H), stored[p + "mlp.up_proj.weight"].float())
    gain = arena.tensors[p + "input_layernorm.gain"]
    assert gain.dtype == torch.float32
    assert torch.equal(gain, stored[p + "input_layernorm.weight"].float() + 1.0)
    assert "lm_head.weight" not in arena.tensors          # tied: the embedding's table serves
    # the seeded source draws the same stored values straight into place
    drawn = place_weights(spec, RandomSource(expected, 4, torch.bfloat16, 0.02, 0.1),
                          torch.float32, "cpu")
    for n in arena.tensors:
        assert torch.equal(arena.tensors[n], drawn.tensors[n]), n
    # an intermediate size that is no multiple of 8: all gates, then all ups
    _, odd = spec_from_config(dict(cfg, intermediate_size=100))
    st = random_tensors(expected_tensors(odd), 1, torch.float32)
    a2 = place_weights(odd, DictSource(st), torch.bfloat16, "cpu")
    gu = a2.tensors["model.layers.0.mlp.gate_up_proj.weight"]
    assert gu.dtype == torch.bfloat16
    assert torch.equal(gu[:100], st["model.layers.0.mlp.gate_proj.weight"].bfloat16())
    assert torch.equal(gu[100:], st["model.layers.0.mlp.up_proj.weight"].bfloat16())
