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
    write_random_model(d, cfg, seed=17, dtype=torch.bfloat16, matrix_std=0.02, norm_std=0.1)
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
