"""Weights on the device: the seeded generator's kernel against its host restatement to
the bit, a model built from a seed against the same model loaded from the folder that
the seed writes, and loading into one buffer without a second copy."""

import pytest
import torch

from helpers import CONFIGS, random_prompts

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_generator_kernel_equals_the_host_formula_bit_for_bit(dtype):
    from strata_inference_b200.kernels import native
    from strata_inference_b200.weights.random_init import (randn_device, randn_host,
                                                           randn_host_range, tensor_key)
    native.require_device(torch.device(DEV))
    for shape, name, std in (((37, 101), "a.weight", 0.02), ((4096,), "b.gain", 0.1),
                             ((300, 80), "model.embed_tokens.weight", 1.0)):
        got = randn_device(shape, 11, name, std, dtype, DEV)
        want = randn_host(shape, 11, name, std, dtype)
        assert torch.equal(got.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                           want.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)), name
    # rows interleaved with another tensor's rows (runs of 8, 16 apart), an offset added after
    # the stored value was rounded to bfloat16, a 32-bit destination
    rows, cols = 64, 24
    dst = torch.zeros(2 * rows, cols, dtype=torch.float32, device=DEV)
    view = dst.as_strided((rows // 8, 8, cols), (16 * cols, cols, 1), 8 * cols)
    native.randn_fill(view, rows, cols, 8, 16, tensor_key(3, "up"), 1.0, 0.1, torch.bfloat16)
    want = randn_host((rows, cols), 3, "up", 0.1, torch.bfloat16).float() + 1.0
    got = dst.view(rows // 8, 2, 8, cols)
    assert torch.equal(got[:, 1].reshape(rows, cols).cpu(), want)
    assert (got[:, 0] == 0).all()
    # far into a large tensor (indices beyond 2^32 / 4): the last elements of 600 M
    n = 600_000_000
    big = randn_device((n,), 5, "big", 0.02, torch.bfloat16, DEV)
    tail = randn_host_range(5, "big", 0.02, n - 4096, 4096, torch.bfloat16)
    assert torch.equal(big[-4096:].cpu().view(torch.int16), tail.view(torch.int16))
    assert abs(big[: 1 << 24].float().std().item() - 0.02) < 2e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_a_seed_names_one_model_on_the_device_and_in_a_folder(tmp_path, name, dtype):
    from strata_inference_b200 import Engine, write_random_model
    cfg = CONFIGS[name]
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    d = write_random_model(str(tmp_path / "m"), cfg, seed=21, dtype=store, matrix_std=0.08,
                           norm_std=0.3)
    on_device = write_random_model(str(tmp_path / "n"), cfg, seed=21, dtype=store, matrix_std=0.08,
                                   norm_std=0.3, device=DEV)
    with open(d + "/model.safetensors", "rb") as f, open(on_device + "/model.safetensors", "rb") as g:
        assert f.read() == g.read()                       # drawn on the host or by the kernel
    loaded = Engine.from_dir(d, dtype=dtype, max_tokens=256)
    drawn = Engine.from_random(cfg, 21, dtype=dtype, max_tokens=256, matrix_std=0.08, norm_std=0.3)
    a, b = loaded.model.arena.tensors, drawn.model.arena.tensors
    assert set(a) == set(b)
    for n in a:
        assert a[n].dtype == b[n].dtype and torch.equal(a[n], b[n]), n
    toks = random_prompts(cfg, [40], seed=2)[0]
    sa, sb = loaded.new_sequence(), drawn.new_sequence()
    assert torch.equal(loaded.step([(sa, toks)], want=[list(range(40))]),
                       drawn.step([(sb, toks)], want=[list(range(40))]))


def test_loading_needs_the_weights_own_bytes_and_one_chunk(tmp_path):
    """Two layers at Gemma2-27B sizes: while the folder is loaded the device never holds
    more than the weight buffer, the cache and one chunk in flight; q|k|v and gate|up
    are written to their fused places straight from the mapped file."""
    from strata_inference_b200 import Engine, write_random_model
    cfg = {
        "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
        "num_hidden_layers": 2, "hidden_size": 4608, "num_attention_heads": 32,
        "num_key_value_heads": 16, "head_dim": 128, "intermediate_size": 36864,
        "vocab_size": 32000, "rope_theta": 10000.0, "sliding_window": 80,
        "query_pre_attn_scalar": 144, "attn_logit_softcapping": 50.0,
        "final_logit_softcapping": 30.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 512,
        "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True,
    }
    d = write_random_model(str(tmp_path / "m"), cfg, seed=7, device=DEV)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    base = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    eng = Engine.from_dir(d, dtype="bfloat16", max_tokens=1024)
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    need = eng.model.weight_bytes() + eng.cache.bytes()
    stored = 2 * (32000 * 4608 + 2 * (4608 * (2 * 32 + 2 * 16) * 128 + 3 * 4608 * 36864))
    assert stored <= eng.model.weight_bytes() <= stored + (1 << 20)
    assert peak <= 1.05 * need, f"peak {peak / 1e9:.2f} GB for {need / 1e9:.2f} GB"
    # and it is the model the seed names
    drawn = Engine.from_random(cfg, 7, dtype="bfloat16", max_tokens=1024)
    toks = random_prompts(cfg, [50], seed=1)[0]
    sa, sb = eng.new_sequence(), drawn.new_sequence()
    assert torch.equal(eng.step([(sa, toks)]), drawn.step([(sb, toks)]))
