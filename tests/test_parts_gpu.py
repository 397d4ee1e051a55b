"""Each part alone against the plain implementation's function for it, and a
toy mixer with state of its own, defined here, registered, built and stepped
without touching the library's files."""

import math

import pytest
import torch

import plain_gemma2 as plain
from helpers import CONFIGS, REL_TOL

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _rt(dtype):
    from strata_inference_b200.parts.base import Runtime
    return Runtime(DEV, dtype)


def _close(got, ref, dtype, what):
    tol = REL_TOL["float32" if dtype == torch.float32 else "bfloat16"]
    got, ref = got.detach().double().cpu(), ref.double().cpu()
    scale = ref.abs().max().item()
    err = (got - ref).abs().max().item()
    assert err <= tol * scale, f"{what}: {err:.3e} vs {tol:.0e} x {scale:.3e}"


def _ctx(rt, cache, seqs, tokens=None):
    """A StepContext for sequences [(slot, start, count)], made the way the engine makes its own."""
    from strata_inference_b200.parts.base import StepContext
    meta = torch.tensor(StepContext.pack(seqs, tokens), dtype=torch.int32, device=DEV)
    return StepContext(meta, seqs, 0, cache, rt)


def _build(part_class, args, stored, rt, *extra):
    from strata_inference_b200.parts.base import build_part
    return build_part(part_class, args, stored, rt, *extra)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from strata_inference_b200.parts.norm import RMSNorm
    rt = _rt(dtype)
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(200, generator=g) * 0.2).to(torch.bfloat16)
    x = torch.randn(7, 200, generator=g)
    for offset in (True, False):
        part = _build(RMSNorm, ({"eps": 1e-4, "unit_offset": offset}, 200), {"weight": w}, rt)
        got = part.forward(x.to(DEV))
        ref = plain.rms_norm(x.double(), w.double() if offset else w.double() - 1.0, 1e-4)
        _close(got, ref, dtype, f"rms_norm part, unit_offset={offset}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    from strata_inference_b200.parts.feed_forward import GatedMLP
    rt = _rt(dtype)
    g = torch.Generator().manual_seed(1)
    for hidden, inter, rows in ((96, 320, 5), (96, 320, 100), (80, 36, 3)):
        ws = {n: (torch.randn(s, generator=g) * 0.2).to(torch.bfloat16) for n, s in (
            ("gate_proj.weight", (inter, hidden)), ("up_proj.weight", (inter, hidden)),
            ("down_proj.weight", (hidden, inter)))}
        part = _build(GatedMLP, ({"intermediate_size": inter, "activation": "gelu_pytorch_tanh"},
                                 hidden), ws, rt)
        x = torch.randn(rows, hidden, generator=g).to(dtype)
        got = part.forward(x.to(DEV), None)
        ref = plain.geglu_ffn(x.double(), ws["gate_proj.weight"].double(),
                              ws["up_proj.weight"].double(), ws["down_proj.weight"].double())
        _close(got, ref, dtype, f"gated_mlp {hidden}x{inter}, {rows} rows")


def _attention_setup(dtype, window, cfg_name="B"):
    from strata_inference_b200.cache.paged import SequenceCache
    from strata_inference_b200.config.spec import PartSpec
    from strata_inference_b200.parts.attention import Attention
    cfg = dict(CONFIGS[cfg_name])
    rt = _rt(dtype)
    g = torch.Generator().manual_seed(2)
    nh, nkv, hd, H = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                      cfg["hidden_size"])
    ws = {"q_proj.weight": torch.randn(nh * hd, H, generator=g) * 0.3,
          "k_proj.weight": torch.randn(nkv * hd, H, generator=g) * 0.3,
          "v_proj.weight": torch.randn(nkv * hd, H, generator=g) * 0.1,
          "o_proj.weight": torch.randn(H, nh * hd, generator=g) * 0.1}
    ws = {k: v.to(torch.bfloat16) for k, v in ws.items()}
    params = {"num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
              "score_scale": cfg["query_pre_attn_scalar"] ** -0.5,
              "logit_softcap": cfg["attn_logit_softcapping"] or 0.0, "window": window,
              "position": PartSpec("rope_neox", {"theta": cfg["rope_theta"], "rotary_dim": hd})}
    part = _build(Attention, (params, H), ws, rt)
    cache = SequenceCache([part.cache_need()], 512, 128, dtype, DEV, page_tokens=8)
    pw = {"self_attn." + k: v for k, v in ws.items()}
    return cfg, rt, part, cache, pw, g


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 16])
def test_attention_part_prompt_then_tokens(dtype, window):
    """The mixer alone: a prompt in one step, then single tokens, against the
    plain attention block over the whole sequence."""
    cfg, rt, part, cache, pw, g = _attention_setup(dtype, window)
    T, cut = 70, 30
    x = torch.randn(T, cfg["hidden_size"], generator=g).to(dtype)
    pcfg = dict(cfg, sliding_window=window or None)
    ref = plain.attention_block(x.double(), {k: v.double() for k, v in pw.items()}, "self_attn.",
                                pcfg, sliding=window > 0)
    slot = cache.acquire()
    other = cache.acquire()      # a neighbour, so that slot 0's pages are not the first ones
    cache.reserve([(other, 9)])
    cache.reserve([(slot, cut)])
    cache.sync_tables()
    got = [part.forward(x[:cut].to(DEV), _ctx(rt, cache, [(slot, 0, cut)]), 0, 0, True)]
    cache.advance(slot, cut)
    for t in range(cut, T):
        cache.reserve([(slot, 1)])
        cache.sync_tables()
        got.append(part.forward(x[t:t + 1].to(DEV), _ctx(rt, cache, [(slot, t, 1)]), 0, 0, True))
        cache.advance(slot, 1)
    _close(torch.cat(got), ref, dtype, f"attention part, window {window}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_reads_a_lent_cache(dtype):
    """A run that borrows another entry's cache projects q only and attends
    over the lender's keys and values."""
    cfg, rt, part, cache, pw, g = _attention_setup(dtype, 0)
    T = 20
    x = torch.randn(T, cfg["hidden_size"], generator=g).to(dtype)
    y = torch.randn(T, cfg["hidden_size"], generator=g).to(dtype)
    slot = cache.acquire()
    cache.reserve([(slot, T)])
    cache.sync_tables()
    ctx = _ctx(rt, cache, [(slot, 0, T)])
    part.forward(x.to(DEV), ctx, 0, 0, True)                 # the lender writes k(x), v(x)
    got = part.forward(y.to(DEV), ctx, 1, 0, False)          # the borrower: q(y) over them
    W = {k: v.double() for k, v in pw.items()}
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    pos = torch.arange(T)
    q = plain.rope_neox((y.double() @ W["self_attn.q_proj.weight"].T).view(T, nh, hd), pos,
                        cfg["rope_theta"])
    k = plain.rope_neox((x.double() @ W["self_attn.k_proj.weight"].T).view(T, nkv, hd), pos,
                        cfg["rope_theta"])
    v = (x.double() @ W["self_attn.v_proj.weight"].T).view(T, nkv, hd)
    o = plain.attention(q, k, v, cfg["query_pre_attn_scalar"] ** -0.5,
                        cfg["attn_logit_softcapping"] or 0.0, 0)
    ref = o.reshape(T, nh * hd) @ W["self_attn.o_proj.weight"].T
    _close(got, ref, dtype, "attention over a lent cache")


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from strata_inference_b200.parts.embedding import LMHead, TokenEmbedding
    rt = _rt(dtype)
    g = torch.Generator().manual_seed(3)
    V, H = 300, 80
    table = (torch.randn(V, H, generator=g) * 0.1).to(torch.bfloat16)
    emb = _build(TokenEmbedding, ({"scale": math.sqrt(H)}, H, V), {"weight": table}, rt)
    toks = torch.randint(0, V, (11,), generator=g, dtype=torch.int32)
    h = emb.forward(_ctx(rt, None, [(0, 0, 11)], toks.tolist()))
    _close(h, plain.embed(toks.tolist(), table.double(), H, torch.float64), torch.float32,
           "embedding")
    for rows in (3, 100):
        y = torch.randn(rows, H, generator=g).to(dtype)
        for cap in (0.0, 2.0):
            head = _build(LMHead, ({"tied": True, "logit_softcap": cap}, H, V), {}, rt, emb)
            got = head.forward(y.to(DEV))
            ref = y.double() @ table.double().T
            if cap:
                ref = cap * torch.tanh(ref / cap)
            assert got.dtype == torch.float32
            _close(got, ref, dtype, f"head, {rows} rows, cap {cap}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    """One sandwich block built from a LayerSpec against the plain decoder layer."""
    from strata_inference_b200.cache.paged import SequenceCache
    from strata_inference_b200.config.registry import spec_from_config
    from strata_inference_b200.engine.model import DecoderModel, expected_tensors
    from strata_inference_b200.weights.random_init import random_tensors
    cfg = dict(CONFIGS["C"], num_hidden_layers=1, layer_types=["sliding_attention"])
    _, spec = spec_from_config(cfg)
    ws = random_tensors(expected_tensors(spec), 5, torch.bfloat16, "cpu", 0.1, 0.3)
    rt = _rt(dtype)
    model = DecoderModel.from_stored(spec, ws, rt)
    cache = SequenceCache(model.cache_needs(), 512, 256, dtype, DEV, page_tokens=16)
    T = 50
    h0 = torch.randn(T, cfg["hidden_size"], generator=torch.Generator().manual_seed(6))
    slot = cache.acquire()
    cache.reserve([(slot, T)])
    cache.sync_tables()
    h = h0.clone().to(DEV)
    model.blocks[0].forward(h, None, _ctx(rt, cache, [(slot, 0, T)]), 0, 0, True, None)
    ref = plain.decoder_layer(h0.double(), {k: v.double() for k, v in ws.items()}, 0, cfg)
    _close(h, ref, dtype, "sandwich block")


# ---------------------------------------------------------------- a toy mixer

class RunningMeanMixer:
    """y_t = W . mean(x_1 .. x_t): needs no keys, only a fixed-size state per
    sequence (the running sum and the count)."""

    @staticmethod
    def tensors(params, hidden):
        from strata_inference_b200.weights.loader import TensorDecl
        return {"mix.weight": TensorDecl((hidden, hidden))}

    def __init__(self, params, hidden, weights, rt):
        self.hidden = hidden
        self.w = weights["mix.weight"].to(device=rt.device, dtype=torch.float32)

    def cache_need(self):
        from strata_inference_b200.cache.paged import CacheNeed, StateNeed
        return CacheNeed(state=StateNeed((self.hidden + 1,), torch.float32))

    def forward(self, x, ctx, entry, cache_entry, owns_cache):
        state = ctx.state(cache_entry)
        out = torch.empty_like(x)
        row = 0
        for slot, n in zip(ctx.slots, ctx.counts):
            xs = x[row:row + n].float()
            sums = torch.cumsum(xs, 0) + state[slot, :-1]
            counts = state[slot, -1] + torch.arange(1, n + 1, device=x.device)
            out[row:row + n] = ((sums / counts[:, None]) @ self.w.t()).to(x.dtype)
            if owns_cache:
                state[slot, :-1] = sums[-1]
                state[slot, -1] = counts[-1]
            row += n
        return out


def _toy_spec(config):
    from strata_inference_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    H = config["hidden_size"]
    norm = PartSpec("rms_norm", {"eps": config["eps"], "unit_offset": False})
    ffn = PartSpec("gated_mlp", {"intermediate_size": config["inter"],
                                 "activation": "gelu_pytorch_tanh"})
    layers = tuple(LayerSpec(prefix=f"layers.{i}.", block="pre_norm",
                             mixer=PartSpec("running_mean", {}), feed_forward=ffn,
                             norms={"pre_mixer": norm, "pre_feed_forward": norm},
                             names={"mixer": "mixer.", "feed_forward": "ffn.",
                                    "pre_mixer": "norm1.", "pre_feed_forward": "norm2."})
                   for i in range(config["layers"]))
    return ModelSpec(architecture="ToyRunningMean", hidden_size=H, vocab_size=config["vocab"],
                     max_positions=config["max_pos"], embedding=PartSpec("token_embedding", {}),
                     layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
                     final_norm=norm, head=PartSpec("lm_head", {"tied": True}),
                     names={"embedding": "embed.", "final_norm": "norm.", "head": "head."})


def _toy_plain(tokens, W, config):
    """The toy model, whole sequence, in 64-bit."""
    eps = config["eps"]
    norm = lambda x, w: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w  # noqa: E731
    h = W["embed.weight"][torch.tensor(tokens)]
    for i in range(config["layers"]):
        p = f"layers.{i}."
        n = norm(h, W[p + "norm1.weight"])
        means = torch.cumsum(n, 0) / torch.arange(1, len(tokens) + 1)[:, None]
        h = h + means @ W[p + "mixer.mix.weight"].T
        n = norm(h, W[p + "norm2.weight"])
        h = h + plain.geglu_ffn(n, W[p + "ffn.gate_proj.weight"], W[p + "ffn.up_proj.weight"],
                                W[p + "ffn.down_proj.weight"])
    return norm(h, W["norm.weight"]) @ W["embed.weight"].T


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    from strata_inference_b200 import Engine, register_architecture, write_random_model
    from strata_inference_b200.parts import register_mixer
    from safetensors.torch import load_file
    register_mixer("running_mean", RunningMeanMixer)
    register_architecture("ToyRunningMean", dict, _toy_spec)
    config = {"architectures": ["ToyRunningMean"], "hidden_size": 40, "inter": 56, "vocab": 90,
              "layers": 2, "eps": 1e-5, "max_pos": 64}
    d = write_random_model(str(tmp_path / "toy"), config, seed=3, dtype=torch.float32,
                           matrix_std=0.2, norm_std=0.5)
    W = {k: v.double() for k, v in load_file(d + "/model.safetensors").items()}
    eng = Engine.from_dir(d, dtype="float32", max_tokens=256)
    assert not eng.cache.groups and len(eng.cache.state) == 2
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, 90, (23,), generator=g).tolist()
    b = torch.randint(0, 90, (9,), generator=g).tolist()
    ref_a, ref_b = _toy_plain(a, W, config), _toy_plain(b, W, config)
    for round_ in range(2):                      # the second round reuses the slots: state is reset
        sa, sb = eng.new_sequence(), eng.new_sequence()
        got = eng.step([(sa, a[:10]), (sb, b[:4])], want=[list(range(10)), list(range(4))])
        _close(got, torch.cat([ref_a[:10], ref_b[:4]]), torch.float32, f"toy prompts {round_}")
        for t in range(4, 9):
            got = eng.step([(sa, [a[6 + t]]), (sb, [b[t]])])
            _close(got, torch.stack([ref_a[6 + t], ref_b[t]]), torch.float32, f"toy step {t}")
        eng.end_sequence(sb)
        got = eng.step([(sa, a[15:])], want=[list(range(8))])
        _close(got, ref_a[15:], torch.float32, f"toy tail {round_}")
        eng.end_sequence(sa)


# ---------------------------------------------------------------- a toy position encoding

class DampedPosition:
    """Not a rotation: q and k are scaled by 1 / (1 + pos * slope_d), a slope per
    dimension.  Has no ``rotary``: the mixer calls ``apply`` before it stores k."""

    @staticmethod
    def tensors(params, head_dim):
        return {}

    def __init__(self, params, head_dim, weights, rt):
        self.slopes = (torch.arange(head_dim, dtype=torch.float32, device=rt.device) + 1) \
            * float(params["slope"]) / head_dim

    def apply(self, q, k, ctx):
        factor = 1.0 / (1.0 + ctx.row_pos.to(torch.float32)[:, None, None] * self.slopes)
        q.copy_((q.float() * factor).to(q.dtype))
        if k is not None:
            k.copy_((k.float() * factor).to(k.dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_position_encoding_through_apply(dtype):
    from strata_inference_b200.cache.paged import SequenceCache
    from strata_inference_b200.config.spec import PartSpec
    from strata_inference_b200.parts import register_position
    from strata_inference_b200.parts.attention import Attention
    register_position("damped", DampedPosition)
    rt = _rt(dtype)
    g = torch.Generator().manual_seed(11)
    H, nh, nkv, hd, slope = 64, 4, 2, 32, 0.05
    ws = {"q_proj.weight": torch.randn(nh * hd, H, generator=g) * 0.2,
          "k_proj.weight": torch.randn(nkv * hd, H, generator=g) * 0.2,
          "v_proj.weight": torch.randn(nkv * hd, H, generator=g) * 0.1,
          "o_proj.weight": torch.randn(H, nh * hd, generator=g) * 0.1}
    ws = {k: v.to(torch.bfloat16) for k, v in ws.items()}
    part = _build(Attention, ({"num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
                               "score_scale": 0.3, "logit_softcap": 0.0, "window": 0,
                               "position": PartSpec("damped", {"slope": slope})}, H), ws, rt)
    cache = SequenceCache([part.cache_need()], 256, 64, dtype, DEV, page_tokens=16)
    T, cut = 40, 25
    x = torch.randn(T, H, generator=g).to(dtype)
    slot = cache.acquire()
    cache.reserve([(slot, cut)])
    cache.sync_tables()
    got = [part.forward(x[:cut].to(DEV), _ctx(rt, cache, [(slot, 0, cut)]), 0, 0, True)]
    cache.advance(slot, cut)
    for t in range(cut, T):
        cache.reserve([(slot, 1)])
        cache.sync_tables()
        got.append(part.forward(x[t:t + 1].to(DEV), _ctx(rt, cache, [(slot, t, 1)]), 0, 0, True))
        cache.advance(slot, 1)
    W = {k: v.double() for k, v in ws.items()}
    factor = 1.0 / (1.0 + torch.arange(T).double()[:, None, None]
                    * (torch.arange(hd).double() + 1) * slope / hd)
    q = (x.double() @ W["q_proj.weight"].T).view(T, nh, hd) * factor
    k = (x.double() @ W["k_proj.weight"].T).view(T, nkv, hd) * factor
    v = (x.double() @ W["v_proj.weight"].T).view(T, nkv, hd)
    ref = plain.attention(q, k, v, 0.3, 0.0, 0).reshape(T, nh * hd) @ W["o_proj.weight"].T
    _close(torch.cat(got), ref, dtype, "attention with a toy position encoding")


# ---------------------------------------------------------------- the schedule is data

def _looped_spec(config):
    """Gemma2's layers run as 0, 1, 0 again (shared weights, a cache of its own),
    then layer 1 again on the keys and values its first run cached."""
    from strata_inference_b200.config.gemma2 import Gemma2Config, gemma2_spec
    from strata_inference_b200.config.spec import ModelSpec, ScheduleEntry
    spec = gemma2_spec(Gemma2Config.from_dict(config))
    fields = dict(spec.__dict__)
    fields["architecture"] = "LoopedGemma2"
    fields["schedule"] = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                          ScheduleEntry(1, cache_of=1))
    return ModelSpec(**fields)


def _looped_plain(tokens, W, cfg):
    eps, T = cfg["rms_norm_eps"], len(tokens)
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    pos = torch.arange(T)
    kept = {}

    def layer(h, i, run, borrow=None):
        p = f"model.layers.{i}."
        n = plain.rms_norm(h, W[p + "input_layernorm.weight"], eps)
        q = plain.rope_neox((n @ W[p + "self_attn.q_proj.weight"].T).view(T, nh, hd), pos,
                            cfg["rope_theta"])
        if borrow is None:
            k = plain.rope_neox((n @ W[p + "self_attn.k_proj.weight"].T).view(T, nkv, hd), pos,
                                cfg["rope_theta"])
            v = (n @ W[p + "self_attn.v_proj.weight"].T).view(T, nkv, hd)
            kept[run] = (k, v)
        else:
            k, v = kept[borrow]
        window = cfg["sliding_window"] if plain.layer_is_sliding(cfg, i) else 0
        o = plain.attention(q, k, v, cfg["query_pre_attn_scalar"] ** -0.5,
                            cfg["attn_logit_softcapping"] or 0.0, window)
        a = o.reshape(T, nh * hd) @ W[p + "self_attn.o_proj.weight"].T
        r = h + plain.rms_norm(a, W[p + "post_attention_layernorm.weight"], eps)
        n2 = plain.rms_norm(r, W[p + "pre_feedforward_layernorm.weight"], eps)
        f = plain.geglu_ffn(n2, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                            W[p + "mlp.down_proj.weight"])
        return r + plain.rms_norm(f, W[p + "post_feedforward_layernorm.weight"], eps)

    h = plain.embed(tokens, W["model.embed_tokens.weight"], cfg["hidden_size"], torch.float64)
    h = layer(h, 0, 0)
    h = layer(h, 1, 1)
    h = layer(h, 0, 2)
    h = layer(h, 1, 3, borrow=1)
    return plain.lm_head(h, W, cfg)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_names_a_layer_twice_and_lends_a_cache(tmp_path, dtype):
    from safetensors.torch import load_file
    from helpers import SHARPEN, assert_logits_close, make_model_dir, random_prompts
    from strata_inference_b200 import Engine, register_architecture
    from strata_inference_b200.config.gemma2 import Gemma2Config
    register_architecture("LoopedGemma2", dict, _looped_spec)
    cfg = dict(CONFIGS["A"], architectures=["LoopedGemma2"], model_type="looped")
    d = make_model_dir(str(tmp_path / "m"), cfg, seed=8, sharpen=SHARPEN[dtype])
    W = {k: v.double() for k, v in load_file(d + "/model.safetensors").items()}
    eng = Engine.from_dir(d, dtype=dtype, max_tokens=512, page_tokens=16)
    assert len(eng.cache.groups) == 2 and sum(len(g.entries) for g in eng.cache.groups) == 3
    # (a run that reads a lent cache reads it by slot: its prompt steps are not recorded and
    # replayed with rows that have no slot)
    assert not eng.model.captures_prompts
    toks = random_prompts(cfg, [60], seed=9)[0]
    ref = _looped_plain(toks, W, cfg)
    slot = eng.new_sequence()
    got = [eng.step([(slot, toks[:35])], want=[list(range(35))])]
    for t in toks[35:]:
        got.append(eng.step([(slot, [t])]))
    eng.end_sequence(slot)
    assert_logits_close(torch.cat(got), ref, dtype, "looped schedule with a lent cache")


# ---------------------------------------------------------------- a toy feed-forward with routing

class TopOneExperts:
    """Each row goes to the expert its router scores highest and comes back scaled by that
    expert's softmax weight: y = p_e * W2_e relu(W1_e x).  Router scores and the softmax are
    32-bit.  Defined here; the framework only learns its name."""

    @staticmethod
    def tensors(params, hidden):
        from strata_inference_b200.weights.loader import TensorDecl
        E, I = params["experts"], params["expert_size"]
        out = {"router.weight": TensorDecl((E, hidden))}
        for e in range(E):
            out[f"experts.{e}.w1.weight"] = TensorDecl((I, hidden))
            out[f"experts.{e}.w2.weight"] = TensorDecl((hidden, I))
        return out

    def __init__(self, params, hidden, weights, rt):
        self.rt = rt
        self.E = params["experts"]
        self.router = weights["router.weight"].to(device=rt.device, dtype=torch.float32)
        self.w1 = [rt.cast_matrix(weights[f"experts.{e}.w1.weight"]) for e in range(self.E)]
        self.w2 = [rt.cast_matrix(weights[f"experts.{e}.w2.weight"]) for e in range(self.E)]

    def forward(self, x, ctx):
        probs = torch.softmax(x.float() @ self.router.t(), dim=-1)
        weight, choice = probs.max(dim=-1)
        out = torch.zeros_like(x)
        for e in range(self.E):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                t = torch.relu(self.rt.linear(x[rows].contiguous(), self.w1[e]))
                y = self.rt.linear(t, self.w2[e]).float() * weight[rows, None]
                out[rows] = y.to(x.dtype)
        return out


def _routed_spec(config):
    """Layer 0: windowed attention and the dense gated feed-forward; layer 1: global attention
    and the routed feed-forward above.  The parts of a layer are chosen layer by layer."""
    from strata_inference_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    H = config["hidden_size"]
    norm = PartSpec("rms_norm", {"eps": config["eps"], "unit_offset": False})
    rope = PartSpec("rope_neox", {"theta": 300.0, "rotary_dim": config["head_dim"]})
    dense = PartSpec("gated_mlp", {"intermediate_size": config["inter"],
                                   "activation": "gelu_pytorch_tanh"})
    routed = PartSpec("top_one_experts", {"experts": config["experts"],
                                          "expert_size": config["expert_size"]})
    layers = []
    for i in range(2):
        mixer = PartSpec("attention", {
            "num_heads": config["heads"], "num_kv_heads": config["kv_heads"],
            "head_dim": config["head_dim"], "score_scale": config["head_dim"] ** -0.5,
            "logit_softcap": 0.0, "window": 6 if i == 0 else 0, "position": rope})
        layers.append(LayerSpec(prefix=f"layers.{i}.", block="pre_norm", mixer=mixer,
                                feed_forward=dense if i == 0 else routed,
                                norms={"pre_mixer": norm, "pre_feed_forward": norm},
                                names={"mixer": "attn.", "feed_forward": "ffn.",
                                       "pre_mixer": "norm1.", "pre_feed_forward": "norm2."}))
    return ModelSpec(architecture="ToyRouted", hidden_size=H, vocab_size=config["vocab"],
                     max_positions=config["max_pos"], embedding=PartSpec("token_embedding", {}),
                     layers=tuple(layers), schedule=(ScheduleEntry(0), ScheduleEntry(1)),
                     final_norm=norm, head=PartSpec("lm_head", {"tied": True}),
                     names={"embedding": "embed.", "final_norm": "norm.", "head": "head."})


def _routed_plain(tokens, W, config):
    """The same model, whole sequence, in 64-bit, from the plain implementation's parts."""
    eps, nh, nkv, hd = config["eps"], config["heads"], config["kv_heads"], config["head_dim"]
    T = len(tokens)
    norm = lambda x, w: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w  # noqa: E731
    pos = torch.arange(T)
    h = W["embed.weight"][torch.tensor(tokens)]
    for i in range(2):
        p = f"layers.{i}."
        n = norm(h, W[p + "norm1.weight"])
        q = plain.rope_neox((n @ W[p + "attn.q_proj.weight"].T).view(T, nh, hd), pos, 300.0)
        k = plain.rope_neox((n @ W[p + "attn.k_proj.weight"].T).view(T, nkv, hd), pos, 300.0)
        v = (n @ W[p + "attn.v_proj.weight"].T).view(T, nkv, hd)
        a = plain.attention(q, k, v, hd ** -0.5, 0.0, 6 if i == 0 else 0)
        h = h + a.reshape(T, nh * hd) @ W[p + "attn.o_proj.weight"].T
        n = norm(h, W[p + "norm2.weight"])
        if i == 0:
            h = h + plain.geglu_ffn(n, W[p + "ffn.gate_proj.weight"], W[p + "ffn.up_proj.weight"],
                                    W[p + "ffn.down_proj.weight"])
        else:
            probs = torch.softmax(n @ W[p + "ffn.router.weight"].T, dim=-1)
            weight, choice = probs.max(dim=-1)
            y = torch.zeros_like(n)
            for r in range(T):
                e = int(choice[r])
                t = torch.relu(W[p + f"ffn.experts.{e}.w1.weight"] @ n[r])
                y[r] = weight[r] * (W[p + f"ffn.experts.{e}.w2.weight"] @ t)
            h = h + y
    return norm(h, W["norm.weight"]) @ W["embed.weight"].T


def test_toy_routed_feed_forward_beside_the_dense_one(tmp_path):
    """A feed-forward with routing, defined in this file, in one layer and the framework's
    dense one in the other: registered, built from a model folder and stepped (prompts of
    unequal lengths, then single tokens) without a change to the framework."""
    from strata_inference_b200 import Engine, register_architecture, write_random_model
    from strata_inference_b200.parts import register_feed_forward
    from safetensors.torch import load_file
    register_feed_forward("top_one_experts", TopOneExperts)
    register_architecture("ToyRouted", dict, _routed_spec)
    config = {"architectures": ["ToyRouted"], "hidden_size": 48, "inter": 40, "vocab": 70,
              "heads": 3, "kv_heads": 1, "head_dim": 16, "experts": 3, "expert_size": 24,
              "eps": 1e-5, "max_pos": 64}
    d = write_random_model(str(tmp_path / "routed"), config, seed=5, dtype=torch.float32,
                           matrix_std=0.3, norm_std=0.5)
    W = {k: v.double() for k, v in load_file(d + "/model.safetensors").items()}
    eng = Engine.from_dir(d, dtype="float32", max_tokens=256)
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, 70, (21,), generator=g).tolist()
    b = torch.randint(0, 70, (8,), generator=g).tolist()
    ref_a, ref_b = _routed_plain(a, W, config), _routed_plain(b, W, config)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    got = eng.step([(sa, a[:12]), (sb, b[:3])], want=[list(range(12)), list(range(3))])
    _close(got, torch.cat([ref_a[:12], ref_b[:3]]), torch.float32, "routed prompts")
    for t in range(3, 8):
        got = eng.step([(sa, [a[9 + t]]), (sb, [b[t]])])
        _close(got, torch.stack([ref_a[9 + t], ref_b[t]]), torch.float32, f"routed step {t}")
    eng.end_sequence(sb)
    got = eng.step([(sa, a[17:])], want=[list(range(4))])
    _close(got, ref_a[17:], torch.float32, "routed tail")
    eng.end_sequence(sa)
    assert eng.cache.pages_in_use() == 0


# ---------------------------------------------------------------- a toy mixer in captured steps

class CapturableRunningMean(RunningMeanMixer):
    """The running-mean mixer with its single-token steps written for capture: the slots
    come from the device tensor ``ctx.seq_slot``, nothing of a step is read on the host."""

    def forward(self, x, ctx, entry, cache_entry, owns_cache):
        if ctx.max_count > 1:
            return super().forward(x, ctx, entry, cache_entry, owns_cache)
        state = ctx.state(cache_entry)
        idx = ctx.seq_slot.long()                    # row b belongs to sequence b
        sums = state[idx, :-1] + x.float()
        counts = state[idx, -1] + 1.0
        if owns_cache:
            state.index_copy_(0, idx, torch.cat([sums, counts[:, None]], dim=1))
        return ((sums / counts[:, None]) @ self.w.t()).to(x.dtype)


def test_toy_mixer_with_state_in_captured_steps_with_changing_slots(tmp_path):
    """Single-token steps replayed from a CUDA graph while the set of slots changes between
    replays: a mixer that indexes its state on the device follows; one that reads the
    step's slots on the host is stopped when the step is first run for capture."""
    from strata_inference_b200 import Engine, register_architecture, write_random_model
    from strata_inference_b200.parts import register_mixer
    from strata_inference_b200.parts.base import CapturedStepError
    from safetensors.torch import load_file
    register_architecture("ToyRunningMean", dict, _toy_spec)
    config = {"architectures": ["ToyRunningMean"], "hidden_size": 40, "inter": 56, "vocab": 90,
              "layers": 2, "eps": 1e-5, "max_pos": 64}
    d = write_random_model(str(tmp_path / "toy"), config, seed=3, dtype=torch.float32,
                           matrix_std=0.2, norm_std=0.5)
    W = {k: v.double() for k, v in load_file(d + "/model.safetensors").items()}
    g = torch.Generator().manual_seed(4)
    reqs = [torch.randint(0, 90, (n,), generator=g).tolist() for n in (30, 22, 26, 19)]
    refs = [_toy_plain(r, W, config) for r in reqs]

    register_mixer("running_mean", RunningMeanMixer)          # loops over ctx.slots on the host
    eng = Engine.from_dir(d, dtype="float32", max_tokens=256)
    s = eng.new_sequence()
    eng.step([(s, reqs[0][:5])])
    eng.decode_step([s], [reqs[0][5]], use_graph=False)       # uncaptured steps may read the host
    with pytest.raises(CapturedStepError, match="slots"):
        eng.decode_step([s], [reqs[0][6]])
    assert eng.length(s) == 6

    register_mixer("running_mean", CapturableRunningMean)
    eng = Engine.from_dir(d, dtype="float32", max_tokens=256)
    slots = [eng.new_sequence() for _ in range(3)]
    pos = [7, 3, 5]
    eng.step([(sl, r[:p]) for sl, r, p in zip(slots, reqs, pos)])
    live = [0, 1, 2]                                          # request index per batch row
    for k in range(12):
        if k == 5:
            # request 1 leaves; request 3 starts in its slot (zeroed state) and joins the
            # same captured step, whose replays now see slots in another order
            eng.end_sequence(slots[1])
            new = eng.new_sequence()
            assert new == slots[1]
            eng.step([(new, reqs[3][:4])])
            slots.append(new)
            pos.append(4)
            live = [3, 0, 2]
        eng.decode_step([slots[i] for i in live], [reqs[i][pos[i]] for i in live])
        ref = torch.stack([refs[i][pos[i]] for i in live])
        _close(eng.last_logits, ref, torch.float32, f"captured toy step {k}")
        for i in live:
            pos[i] += 1
    assert eng.recorded_step(3).graph is not None    # the steps were replays


# ---------------------------------------------------------------- a toy embedding with positions

class LearnedPositionEmbedding:
    """h = table[token] + positions[absolute position]: an embedding that needs the step's
    positions, which it gets because embeddings are given the whole step context."""

    @staticmethod
    def tensors(params, hidden, vocab):
        from strata_inference_b200.weights.loader import TensorDecl
        return {"weight": TensorDecl((vocab, hidden)),
                "positions.weight": TensorDecl((params["max_positions"], hidden))}

    def __init__(self, params, hidden, vocab, weights, rt):
        self.table = rt.cast_matrix(weights["weight"])        # (a tied head reads `table`)
        self.positions = weights["positions.weight"].to(device=rt.device, dtype=torch.float32)

    def forward(self, ctx):
        return self.table[ctx.tokens.long()].float() + self.positions[ctx.row_pos.long()]


def _learned_pos_spec(config):
    from strata_inference_b200.config.spec import ModelSpec, PartSpec
    spec = _toy_spec(config)
    fields = dict(spec.__dict__)
    fields["architecture"] = "ToyLearnedPositions"
    fields["embedding"] = PartSpec("learned_positions", {"max_positions": config["max_pos"]})
    return ModelSpec(**fields)


def test_toy_embedding_with_learned_positions(tmp_path):
    from strata_inference_b200 import Engine, register_architecture, write_random_model
    from strata_inference_b200.parts import register_embedding, register_mixer
    from safetensors.torch import load_file
    register_mixer("running_mean", CapturableRunningMean)
    register_embedding("learned_positions", LearnedPositionEmbedding)
    register_architecture("ToyLearnedPositions", dict, _learned_pos_spec)
    config = {"architectures": ["ToyLearnedPositions"], "hidden_size": 40, "inter": 56,
              "vocab": 90, "layers": 1, "eps": 1e-5, "max_pos": 48}
    d = write_random_model(str(tmp_path / "toy"), config, seed=6, dtype=torch.float32,
                           matrix_std=0.2, norm_std=0.5)
    W = {k: v.double() for k, v in load_file(d + "/model.safetensors").items()}
    assert W["embed.positions.weight"].shape == (48, 40)
    toks = torch.randint(0, 90, (30,), generator=torch.Generator().manual_seed(7)).tolist()
    # the plain toy model with the positions added to the embedded tokens
    shifted = dict(W)
    eps = config["eps"]
    norm = lambda x, w: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w  # noqa: E731
    h = W["embed.weight"][torch.tensor(toks)] + W["embed.positions.weight"][:30]
    n = norm(h, W["layers.0.norm1.weight"])
    h = h + (torch.cumsum(n, 0) / torch.arange(1, 31)[:, None]) @ W["layers.0.mixer.mix.weight"].T
    n = norm(h, W["layers.0.norm2.weight"])
    h = h + plain.geglu_ffn(n, W["layers.0.ffn.gate_proj.weight"], W["layers.0.ffn.up_proj.weight"],
                            W["layers.0.ffn.down_proj.weight"])
    ref = norm(h, W["norm.weight"]) @ W["embed.weight"].T
    del shifted
    eng = Engine.from_dir(d, dtype="float32", max_tokens=128)
    s = eng.new_sequence()
    got = [eng.step([(s, toks[:12])], want=[list(range(12))])]
    for t in toks[12:]:
        eng.decode_step([s], [t])                 # captured from the second one on
        got.append(eng.last_logits.clone())
    _close(torch.cat(got), ref, torch.float32, "learned positions, prompt then captured steps")
