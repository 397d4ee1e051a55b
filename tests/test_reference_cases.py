"""The reference's own unit-test cases, run on the plain implementation.

strata-inference is a Rust crate; where these tests run it can be neither imported nor
compiled, so the plain implementation (tests/plain_gemma2.py) cannot be compared with its
binaries.  What can be taken from it is what its unit tests assert: each case below is an
input and an expectation from one ``#[test]`` of the project (file and lines given), with
the project's own tolerance, applied to the plain implementation's function for that
operation.  The cases are data; nothing of the project's code is restated here.
"""

import math

import torch

import plain_gemma2 as plain

F64 = torch.float64


def _gain(w):
    """The reference's norm weight is the gain itself; the plain function takes w with
    gain = 1 + w."""
    return torch.tensor(w, dtype=F64) - 1.0


def test_rms_norm_cases():
    # src/backend/cpu.rs:1853-1875 test_rms_norm_basic
    out = plain.rms_norm(torch.tensor([[1.0, 2.0, 3.0, 4.0]], dtype=F64), _gain([1.0] * 4), 1e-5)
    rms = math.sqrt(7.5 + 1e-5)
    for i in range(4):
        assert abs(out[0, i].item() - (i + 1.0) / rms) < 1e-4
    # src/backend/cpu.rs:1878-1890 test_rms_norm_with_weight
    out = plain.rms_norm(torch.tensor([[3.0, 4.0]], dtype=F64), _gain([2.0, 0.5]), 1e-5)
    inv = 1.0 / math.sqrt(12.5 + 1e-5)
    assert abs(out[0, 0].item() - 3.0 * inv * 2.0) < 1e-4
    assert abs(out[0, 1].item() - 4.0 * inv * 0.5) < 1e-4
    # src/backend/cpu.rs:1893-1906 test_rms_norm_multi_row
    out = plain.rms_norm(torch.tensor([[1.0, 1.0], [2.0, 2.0]], dtype=F64), _gain([1.0, 1.0]), 0.0)
    assert (out - 1.0).abs().max().item() < 1e-5


def test_geglu_cases():
    # src/backend/cpu.rs:3387-3416 test_geglu_basic
    gate = torch.tensor([-1.0, 0.0, 1.0, 2.0], dtype=F64)
    up = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=F64)
    out = plain.gelu_tanh(gate) * up
    assert abs(out[0].item() - (-0.1588)) < 0.01
    assert abs(out[1].item()) < 1e-6
    assert abs(out[2].item() - 0.8412 * 3.0) < 0.05
    assert abs(out[3].item() - 1.9545 * 4.0) < 0.05
    # src/backend/cpu.rs:3419-3428 test_geglu_zero_up
    out = plain.gelu_tanh(torch.tensor([1.0, 2.0, 3.0], dtype=F64)) * torch.zeros(3, dtype=F64)
    assert out.abs().max().item() < 1e-6


def test_rope_neox_cases():
    # src/backend/cpu.rs:3430-3447 test_rope_neox_basic: position 0 changes nothing
    q = torch.tensor([1.0, 0.0, 0.0, 0.0], dtype=F64).view(1, 1, 4)
    k = torch.tensor([0.0, 1.0, 0.0, 0.0], dtype=F64).view(1, 1, 4)
    pos0 = torch.tensor([0])
    assert abs(plain.rope_neox(q, pos0, 10000.0)[0, 0, 0].item() - 1.0) < 1e-5
    assert abs(plain.rope_neox(k, pos0, 10000.0)[0, 0, 1].item() - 1.0) < 1e-5
    # src/backend/cpu.rs:3450-3493 test_rope_neox_preserves_norm: 2 rows, 2 heads of 4, from
    # position 3 on
    qd = torch.tensor([i * 0.1 + 0.1 for i in range(16)], dtype=F64).view(2, 2, 4)
    kd = torch.tensor([i * 0.05 + 0.5 for i in range(16)], dtype=F64).view(2, 2, 4)
    pos = torch.tensor([3, 4])
    for x in (qd, kd):
        y = plain.rope_neox(x, pos, 10000.0)
        assert (y.norm(dim=-1) - x.norm(dim=-1)).abs().max().item() < 1e-4
    # src/backend/cpu.rs:3496-3520 test_rope_neox_differs_from_rope: half-split pairs, not
    # neighbours; the interleaved rotation of [1, 2, 3, 4] at position 5 pairs (1, 2), (3, 4)
    x = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=F64).view(1, 1, 4)
    y = plain.rope_neox(x, torch.tensor([5]), 10000.0).flatten()
    a0, a1 = 5.0, 5.0 * 10000.0 ** -0.5
    inter = [math.cos(a0) - 2 * math.sin(a0), math.sin(a0) + 2 * math.cos(a0),
             3 * math.cos(a1) - 4 * math.sin(a1), 3 * math.sin(a1) + 4 * math.cos(a1)]
    assert max(abs(y[i].item() - inter[i]) for i in range(4)) > 1e-6
    half = [math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            math.sin(a0) + 3 * math.cos(a0), 2 * math.sin(a1) + 4 * math.cos(a1)]
    assert max(abs(y[i].item() - half[i]) for i in range(4)) < 1e-5


def _decode(q, k, v, total_len, nh, nkv, hd, scale, cap):
    """One query over `total_len` cached positions, as grouped_attention_decode is called
    in the reference's tests: the query is the last position of a whole sequence."""
    qs = torch.zeros(total_len, nh, hd, dtype=F64)
    qs[-1] = torch.tensor(q, dtype=F64).view(nh, hd)
    ks = torch.tensor(k, dtype=F64).view(total_len, nkv, hd)
    vs = torch.tensor(v, dtype=F64).view(total_len, nkv, hd)
    return plain.attention(qs, ks, vs, scale, cap, 0)[-1].flatten()


def test_decode_attention_cases():
    # src/backend/cpu.rs:3565-3610 test_grouped_attention_decode_basic: finite values
    out = _decode([1.0, 0.0, 0.0, 1.0],
                  [1.0, 0.0, 0.0, 1.0, 0.0, 1.0, 1.0, 0.0, 1.0, 1.0, 1.0, 1.0],
                  [1.0, 0.0, 0.0, 1.0, 0.0, 1.0, 1.0, 0.0, 0.5, 0.5, 0.5, 0.5],
                  3, 2, 2, 2, 1.0 / math.sqrt(2.0), 0.0)
    assert out.shape == (4,) and torch.isfinite(out).all()
    # src/backend/cpu.rs:3613-3668 test_grouped_attention_decode_gqa: heads 0, 1 read kv head 0,
    # heads 2, 3 kv head 1; head 0 (q = [1, 0]) scores [1, 0] and attends more to position 0
    out = _decode([1.0, 0.0, 0.0, 1.0, 1.0, 1.0, -1.0, 0.0],
                  [1.0, 0.0, 0.0, 1.0, 0.0, 1.0, 1.0, 0.0],
                  [1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0], 2, 4, 2, 2, 1.0 / math.sqrt(2.0), 0.0)
    assert out.shape == (8,) and torch.isfinite(out).all()
    p0 = math.exp(1 / math.sqrt(2)) / (math.exp(1 / math.sqrt(2)) + 1.0)
    assert p0 > 0.5 and abs(out[0].item() - (p0 * 1.0 + (1 - p0) * 5.0)) < 1e-9
    # head 3 (q = [-1, 0]) reads kv head 1: scores [0, -1], values [3, 4] and [7, 8]
    assert abs(out[7].item() - (p0 * 4.0 + (1 - p0) * 8.0)) < 1e-9
    # src/backend/cpu.rs:3671-3725 test_grouped_attention_decode_softcap: a cap of 1 makes the
    # weights more uniform
    args = ([10.0, 10.0], [10.0, 10.0, -10.0, -10.0], [1.0, 0.0, 0.0, 1.0], 2, 1, 1, 2, 1.0)
    free, capped = _decode(*args, 0.0), _decode(*args, 1.0)
    assert abs(capped[0] - capped[1]) < abs(free[0] - free[1])
    # src/backend/cpu.rs:3728-3743 test_grouped_attention_decode_single_token: one position
    # gets all the weight
    out = _decode([1.0, 2.0, 3.0, 4.0], [0.5] * 4, [10.0, 20.0, 30.0, 40.0], 1, 2, 2, 2,
                  1.0 / math.sqrt(2.0), 0.0)
    assert (out - torch.tensor([10.0, 20.0, 30.0, 40.0], dtype=F64)).abs().max().item() < 1e-5


def test_sampler_cases():
    S = plain.sample_token
    rng = plain.XorShift64
    # src/engine/sampler.rs:158-174 argmax
    assert plain.argmax([1.0, 3.0, 2.0]) == 1 and plain.argmax([5.0, 1.0, 2.0]) == 0
    assert plain.argmax([1.0, 2.0, 5.0]) == 2 and plain.argmax([-3.0, -1.0, -2.0]) == 1
    assert plain.argmax([42.0]) == 0
    # :176-200 greedy ignores the generator
    logits = torch.tensor([1.0, 5.0, 2.0, 3.0])
    assert S(logits, 0.0, 0, 1.0, rng(42)) == 1 == S(logits, 0.0, 0, 1.0, rng(99))
    # :202-218 the same seed gives the same token
    assert S(logits, 1.0, 0, 1.0, rng(42)) == S(logits, 1.0, 0, 1.0, rng(42))
    # :220-233 top_k = 1 keeps the best token only
    assert S(torch.tensor([1.0, 10.0, 2.0, 3.0]), 1.0, 1, 1.0, rng(42)) == 1
    # :235-247 a tiny top_p keeps the best token only
    assert S(torch.tensor([0.0, 100.0, 0.0, 0.0]), 1.0, 0, 0.01, rng(42)) == 1
    # :249-275 a low temperature favours the top token: more than 90 of 100 draws
    r = rng(42)
    assert sum(S(torch.tensor([1.0, 2.0, 3.0, 4.0]), 0.01, 0, 1.0, r) == 3 for _ in range(100)) > 90
    # :277-294 top_k = 2 with top_p = 0.5 picks among the two best
    assert S(torch.tensor([1.0, 10.0, 9.0, 0.0]), 1.0, 2, 0.5, rng(42)) in (1, 2)
    # :296-313 the generator moves on, and its floats lie in [0, 1)
    r = rng(42)
    a, b, c = r.next_u64(), r.next_u64(), r.next_u64()
    assert a != b and b != c
    r = rng(42)
    assert all(0.0 <= r.next_f32() < 1.0 for _ in range(1000))
    # :315-320 no logits: token 0;  :322-337 every draw is a valid index
    assert S(torch.tensor([]), 0.0, 0, 1.0, rng(42)) == 0
    r = rng(42)
    assert all(0 <= S(torch.ones(100), 1.0, 0, 1.0, r) < 100 for _ in range(100))
