"""The engine at the layer sizes of Gemma2-2B (hidden 2304, 8 heads of 256 in
4 groups, intermediate 9216, vocabulary 256000) and of Gemma2-27B (hidden 4608,
32 heads of 128 in 16 groups, intermediate 36864), two layers deep, against the
plain implementation: whole prompt, last tokens one by one, unequal batch.
The tiny configurations never reach the code paths that these sizes select
(head size 256, the 16-byte vector paths, the cluster split of the products,
the tensor-memory product for many rows of logits)."""

import pytest
import torch

import plain_gemma2 as plain
from helpers import REL_TOL, plain_weights, random_prompts

pytestmark = pytest.mark.gpu

CFG_2B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 2304, "num_attention_heads": 8,
    "num_key_value_heads": 4, "head_dim": 256, "intermediate_size": 9216, "vocab_size": 256000,
    "rope_theta": 10000.0, "sliding_window": 96, "query_pre_attn_scalar": 256,
    "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 512, "hidden_activation": "gelu_pytorch_tanh",
    "tie_word_embeddings": True,
}
# the layer sizes of Gemma2-27B (32 heads of 128 in 16 groups) with a shorter vocabulary,
# which keeps the plain implementation's 32-bit weights to a few GB
CFG_27B = dict(CFG_2B, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16,
               head_dim=128, intermediate_size=36864, vocab_size=32000, query_pre_attn_scalar=144,
               sliding_window=80)
CONFIGS = {"2b": CFG_2B, "27b": CFG_27B}


def _rel(got, ref):
    got, ref = got.detach().float().cpu(), ref.float()
    return (got - ref).abs().max().item() / ref.abs().max().item()


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    """The model folder, the requests and the plain logits, shared by both types."""
    from strata_inference_b200.weights.random_init import write_random_model
    cfg = CONFIGS[request.param]
    d = str(tmp_path_factory.mktemp("gemma2_%s_sizes" % request.param))
    write_random_model(d, cfg, seed=17, dtype=torch.bfloat16, matrix_std=0.02, norm_std=0.1,
                       device="cuda:0")
    W = {k: v.float() for k, v in plain_weights(d).items()}
    reqs = random_prompts(cfg, [200, 37, 150], seed=18)
    refs = [plain.forward(t, W, cfg, dtype=torch.float32) for t in reqs]
    return d, reqs, refs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_layers_of_real_sizes(model, dtype):
    from strata_inference_b200 import Engine
    d, reqs, refs = model
    tol = REL_TOL[dtype]
    eng = Engine.from_dir(d, dtype=dtype, max_tokens=1024)
    # whole, every position wanted (more than 16 rows of logits)
    s = eng.new_sequence()
    got = eng.step([(s, reqs[0])], want=[list(range(len(reqs[0])))])
    eng.end_sequence(s)
    assert _rel(got, refs[0]) <= tol, f"whole prompt: {_rel(got, refs[0]):.2e}"
    # prefix, then the last 32 tokens one by one (crosses the window of 96 and a page edge)
    s = eng.new_sequence()
    cut = len(reqs[0]) - 32
    outs = [eng.step([(s, reqs[0][:cut])])]
    for t in reqs[0][cut:]:
        outs.append(eng.step([(s, [t])]))
    eng.end_sequence(s)
    err = _rel(torch.cat(outs), refs[0][cut - 1:])
    assert err <= tol, f"last 32 one by one: {err:.2e}"
    # an unequal batch, then 5 single-token steps; the short request ends after 3
    prompt = [120, 30, 100]
    slots = [eng.new_sequence() for _ in reqs]
    got = eng.step([(sl, r[:p]) for sl, r, p in zip(slots, reqs, prompt)])
    ref = torch.stack([f[p - 1] for f, p in zip(refs, prompt)])
    assert _rel(got, ref) <= tol, f"batch prompts: {_rel(got, ref):.2e}"
    live = [0, 1, 2]
    for k in range(5):
        if k == 3:
            eng.end_sequence(slots[1])
            live = [0, 2]
        got = eng.step([(slots[i], [reqs[i][prompt[i] + k]]) for i in live])
        ref = torch.stack([refs[i][prompt[i] + k] for i in live])
        assert _rel(got, ref) <= tol, f"batch step {k}: {_rel(got, ref):.2e}"
    for i in live:
        eng.end_sequence(slots[i])
    assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_of_4096_at_real_sizes(tmp_path, dtype):
    """Two layers at Gemma2-2B sizes with the real window of 4096: a 4 100-token prompt (the
    paired tcgen05 prompt kernel with a window; the sliding layer's ring of 4 160 positions
    is written around once), then 150 single-token steps that take the ring over its end.
    The plain implementation runs on the GPU here (its code is the same; 4 250 x 4 250 scores
    per head are too slow on the host)."""
    from strata_inference_b200 import Engine
    from strata_inference_b200.weights.random_init import write_random_model
    cfg = dict(CFG_2B, vocab_size=32000, sliding_window=4096, max_position_embeddings=8192)
    d = str(tmp_path / "gemma2_window")
    write_random_model(d, cfg, seed=3, dtype=torch.bfloat16, matrix_std=0.02, norm_std=0.1,
                       device="cuda:0")
    toks = random_prompts(cfg, [4250], seed=4)[0]
    with torch.no_grad(), torch.device("cuda"):
        W = {k: v.float().cuda() for k, v in plain_weights(d).items()}
        ref = plain.forward(toks, W, cfg, dtype=torch.float32).cpu()
    del W
    eng = Engine.from_dir(d, dtype=dtype, max_tokens=8192)
    s = eng.new_sequence()
    outs = [eng.step([(s, toks[:4100])], want=[[4098, 4099]])]
    for t in toks[4100:]:
        outs.append(eng.step([(s, [t])]))
    eng.end_sequence(s)
    err = _rel(torch.cat(outs), ref[4098:])
    assert err <= REL_TOL[dtype], f"window of 4096, {dtype}: {err:.2e}"
