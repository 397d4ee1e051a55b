"""The plain implementation itself, on cases small enough to check by hand,
after the reference's own unit tests of its CPU operations
(src/backend/cpu.rs:1853-1906 rms_norm, :3387-3428 geglu, :3430-3550 rope_neox,
:3566-3743 decode attention; src/engine/sampler.rs:158-337 sampler;
src/model/layer.rs:2554-2604 cached == uncached)."""

import math

import pytest
import torch

import plain_gemma2 as plain
from helpers import TINY_A, TINY_B, make_model_dir, plain_weights, random_prompts

F64 = torch.float64


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    w = torch.tensor([0.0, 1.0], dtype=F64)           # gains 1 and 2
    out = plain.rms_norm(x, w, 0.0)
    r = 1.0 / math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[3 * r, 8 * r]], dtype=F64))
    assert torch.allclose(plain.rms_norm(torch.zeros(1, 4, dtype=F64), torch.zeros(4, dtype=F64), 1e-6),
                          torch.zeros(1, 4, dtype=F64))


def test_gelu_tanh_values():
    g = torch.tensor([0.0, 1.0, -1.0, 3.0], dtype=F64)
    want = [0.0, 0.8411919906082768, -0.15880800939172324, 2.9963627438855624]
    assert torch.allclose(plain.gelu_tanh(g), torch.tensor(want, dtype=F64), atol=1e-12)


def test_rope_half_split_pairs_and_preserves_norms():
    x = torch.randn(5, 2, 8, dtype=F64, generator=torch.Generator().manual_seed(0))
    pos = torch.tensor([0, 1, 2, 7, 100])
    y = plain.rope_neox(x, pos, 10000.0)
    assert torch.equal(y[0], x[0])                                   # position 0: no rotation
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # dimension i pairs with i + 4 at angle pos * theta^(-2i/8)
    i, p = 1, 7
    ang = p * 10000.0 ** (-2 * i / 8)
    a, b = x[3, 0, i], x[3, 0, i + 4]
    assert torch.allclose(y[3, 0, i], a * math.cos(ang) - b * math.sin(ang), atol=1e-6)
    assert torch.allclose(y[3, 0, i + 4], a * math.sin(ang) + b * math.cos(ang), atol=1e-6)
    # relative positions: <rope(q,m), rope(k,n)> depends on m - n only
    q, k = x[:1, :1], x[1:2, :1]
    d1 = (plain.rope_neox(q, torch.tensor([5]), 1e4) * plain.rope_neox(k, torch.tensor([3]), 1e4)).sum()
    d2 = (plain.rope_neox(q, torch.tensor([45]), 1e4) * plain.rope_neox(k, torch.tensor([43]), 1e4)).sum()
    assert torch.allclose(d1, d2, atol=1e-5)


def test_attention_masks_and_groups():
    g = torch.Generator().manual_seed(1)
    T = 6
    q = torch.randn(T, 4, 8, dtype=F64, generator=g)
    k = torch.randn(T, 2, 8, dtype=F64, generator=g)
    v = torch.randn(T, 2, 8, dtype=F64, generator=g)
    out = plain.attention(q, k, v, 0.5, 0.0, 0)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])  # first row sees itself
    # heads 0,1 share kv head 0; heads 2,3 share kv head 1
    s = (q[5, 2] @ k[:, 1].T) * 0.5
    want = torch.softmax(s, 0) @ v[:, 1]
    assert torch.allclose(out[5, 2], want)
    # a window of 2: row 5 sees keys 4 and 5 only
    outw = plain.attention(q, k, v, 0.5, 0.0, 2)
    want = torch.softmax(s[4:6], 0) @ v[4:6, 1]
    assert torch.allclose(outw[5, 2], want)
    assert torch.allclose(outw[1], out[1])                           # still inside the window
    # soft cap bounds the scores: with a tiny cap attention becomes uniform
    outc = plain.attention(q, k, v, 0.5, 1e-9, 0)
    assert torch.allclose(outc[5, 0], v[:, 0].mean(0), atol=1e-6)


def test_zero_feed_forward_and_attention_leave_the_residual(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_A, seed=1)
    W = {k: v.double() for k, v in plain_weights(d).items()}
    for n in W:
        if n.endswith("down_proj.weight") or n.endswith("o_proj.weight"):
            W[n] = torch.zeros_like(W[n])
    h = torch.randn(5, TINY_A["hidden_size"], dtype=F64, generator=torch.Generator().manual_seed(2))
    assert torch.allclose(plain.decoder_layer(h, W, 0, TINY_A), h)


def test_logits_of_a_prefix_do_not_change_when_tokens_follow(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_B, seed=2)
    W = plain_weights(d)
    toks = random_prompts(TINY_B, [30], seed=3)[0]
    full = plain.forward(toks, W, TINY_B)
    part = plain.forward(toks[:17], W, TINY_B)
    assert torch.allclose(full[:17], part, atol=1e-10)
    with pytest.raises(ValueError, match="exceeds vocab_size"):
        plain.forward([TINY_B["vocab_size"]], W, TINY_B)
    toks_a = random_prompts(TINY_A, [30], seed=3)[0]
    capped = plain.forward(toks_a, plain_weights(make_model_dir(str(tmp_path / "a"), TINY_A, 1)), TINY_A)
    assert capped.abs().max() < TINY_A["final_logit_softcapping"]


def test_xorshift_and_sampler():
    rng = plain.XorShift64(0)
    assert rng.state == 1                                            # seed 0 becomes 1
    a = plain.XorShift64(42)
    b = plain.XorShift64(42)
    assert [a.next_u64() for _ in range(5)] == [b.next_u64() for _ in range(5)]
    x = 42
    x ^= (x << 13) & (2 ** 64 - 1); x ^= x >> 7; x ^= (x << 17) & (2 ** 64 - 1)
    assert plain.XorShift64(42).next_u64() == x
    assert all(0.0 <= plain.XorShift64(s).next_f32() < 1.0 for s in range(1, 50))
    logits = torch.tensor([1.0, 3.0, 2.0, 3.0])
    assert plain.argmax(logits.tolist()) == 1                        # first maximum
    assert plain.sample_token(logits, 0.0, 0, 1.0, plain.XorShift64(1)) == 1
    # top_k = 1 is greedy whatever the draw; top_p tiny keeps the best token only
    for seed in range(1, 20):
        assert plain.sample_token(logits, 1.0, 1, 1.0, plain.XorShift64(seed)) == 1
        assert plain.sample_token(torch.tensor([0.0, 5.0, 1.0]), 1.0, 0, 0.1, plain.XorShift64(seed)) == 1
    # the distribution follows the softmax
    rng = plain.XorShift64(7)
    draws = [plain.sample_token(torch.tensor([0.0, math.log(3.0)]), 1.0, 0, 1.0, rng) for _ in range(4000)]
    assert abs(sum(draws) / 4000 - 0.75) < 0.03
    # top_k excludes everything below the k best
    rng = plain.XorShift64(9)
    big = torch.tensor([0.1 * i for i in range(50)])
    assert all(plain.sample_token(big, 5.0, 3, 1.0, rng) >= 47 for _ in range(200))


def test_generate_stop_rules(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_A, seed=4)
    W = plain_weights(d)
    prompt = random_prompts(TINY_A, [4], seed=5)[0]
    free, reason = plain.generate(prompt, W, TINY_A, 6)
    assert len(free) == 6 and reason == "max_tokens"
    out, reason = plain.generate(prompt, W, TINY_A, 6, stop_tokens=[free[2]])
    assert out == free[:free.index(free[2])] and reason == "eos"
    out, reason = plain.generate(prompt, W, TINY_A, 100, max_seq_len=7)
    assert len(out) == 4 and reason == "context_length" and out == free[:4]
    assert plain.generate(prompt, W, TINY_A, 0) == ([], "max_tokens")
    with pytest.raises(ValueError):
        plain.generate([], W, TINY_A, 1)
    with pytest.raises(ValueError):
        plain.generate([1] * 7, W, TINY_A, 1, max_seq_len=7)
