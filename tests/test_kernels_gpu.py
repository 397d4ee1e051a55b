"""Each kernel alone against a plain PyTorch restatement of the same
operation in 32-bit/64-bit, at sizes other than the engine tests use."""

import math
import os

import pytest
import torch

import plain_gemma2 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _native():
    from strata_inference_b200.kernels import native
    native.require_device(torch.device(DEV))
    return native


def _tol(dtype):
    return 2e-6 if dtype == torch.float32 else 1e-2


def _close(got, ref, dtype, what, factor=1.0):
    got = got.detach().double().cpu()
    ref = ref.double().cpu()
    scale = max(ref.abs().max().item(), 1e-30)
    err = (got - ref).abs().max().item()
    assert err <= factor * _tol(dtype) * scale, f"{what}: {err:.3e} vs scale {scale:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,vocab", [(72, 50), (2304, 1000)])
def test_embed_rows(dtype, hidden, vocab):
    n = _native()
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, hidden, generator=g).to(dtype)
    toks = torch.randint(0, vocab, (37,), generator=g, dtype=torch.int32)
    out = torch.empty(37, hidden, dtype=torch.float32, device=DEV)
    n.embed_rows(toks.to(DEV), table.to(DEV), math.sqrt(hidden), out)
    ref = plain.embed(toks.tolist(), table.double(), hidden, torch.float64)
    _close(out, ref, torch.float32, "embed_rows")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [48, 256, 1000, 2304, 4608, 20000])
@pytest.mark.parametrize("rows", [9, 600])
def test_rms_norm_and_fused_add(dtype, hidden, rows):
    n = _native()
    g = torch.Generator().manual_seed(1)
    h = torch.randn(rows, hidden, generator=g) * 3
    a = torch.randn(rows, hidden, generator=g).to(dtype)
    w1 = torch.randn(hidden, generator=g) * 0.3
    w2 = torch.randn(hidden, generator=g) * 0.3
    eps1, eps2 = 1e-5, 3e-3
    # norm of selected rows of a 32-bit stream
    idx = torch.tensor([8, 0, 3], dtype=torch.int32)
    out = torch.empty(3, hidden, dtype=dtype, device=DEV)
    n.rms_norm(h.to(DEV), (1 + w1).to(DEV), eps1, out, idx.to(DEV))
    _close(out, plain.rms_norm(h.double()[idx.long()], w1.double(), eps1), dtype, "rms_norm rows")
    # norm of an activation-typed input into 32-bit
    out32 = torch.empty(rows, hidden, dtype=torch.float32, device=DEV)
    n.rms_norm(a.to(DEV), (1 + w2).to(DEV), eps2, out32)
    _close(out32, plain.rms_norm(a.double(), w2.double(), eps2), torch.float32, "rms_norm act")
    # h += rms(a) g1 ; out = rms(h) g2
    hd = h.clone().to(DEV)
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    n.add_rms_norm(a.to(DEV), (1 + w1).to(DEV), eps1, hd, (1 + w2).to(DEV), eps2, out)
    h_ref = h.double() + plain.rms_norm(a.double(), w1.double(), eps1)
    _close(hd, h_ref, torch.float32, "add_rms_norm residual")
    _close(out, plain.rms_norm(h_ref, w2.double(), eps2), dtype, "add_rms_norm out")
    # without a post norm and without a following norm
    hd = h.clone().to(DEV)
    n.add_rms_norm(a.to(DEV), None, 0.0, hd, None, 0.0, None)
    _close(hd, h.double() + a.double(), torch.float32, "plain residual add")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter,group", [(24, 0), (24, 8), (1000, 8), (9, 0)])
def test_gelu_mul(dtype, inter, group):
    n = _native()
    g = torch.Generator().manual_seed(2)
    gate = (torch.randn(5, inter, generator=g) * 2).to(dtype)
    up = torch.randn(5, inter, generator=g).to(dtype)
    if group:
        gu = torch.cat([gate.view(5, -1, group), up.view(5, -1, group)], dim=2).reshape(5, -1)
    else:
        gu = torch.cat([gate, up], dim=1)
    out = torch.empty(5, inter, dtype=dtype, device=DEV)
    n.gelu_mul(gu.contiguous().to(DEV), out, group)
    _close(out, plain.gelu_tanh(gate.double()) * up.double(), dtype, "gelu_mul")


def test_softcap():
    n = _native()
    x = torch.linspace(-200, 200, 10001)
    y = n.softcap_(x.clone().to(DEV), 30.0)
    _close(y, 30.0 * torch.tanh(x.double() / 30.0), torch.float32, "softcap")


def _paged(k, v, page_tokens, ring_tokens, n_kv, hd, dtype, positions):
    """Lay keys/values [T, n_kv, hd] of ONE sequence out as pages in shuffled
    order; returns pools and the page table for slot 1 of 3."""
    T = k.shape[0]
    cells = ring_tokens if ring_tokens else -(-T // page_tokens) * page_tokens
    n_seq_pages = cells // page_tokens
    n_pages = n_seq_pages + 5
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(9))[:n_seq_pages]
    kp = torch.full((n_pages, n_kv, page_tokens, hd), float("nan"), dtype=dtype)
    vp = torch.full((n_pages, n_kv, page_tokens, hd), float("nan"), dtype=dtype)
    for p in positions:
        cell = p % ring_tokens if ring_tokens else p
        kp[perm[cell // page_tokens], :, cell % page_tokens] = k[p].to(dtype)
        vp[perm[cell // page_tokens], :, cell % page_tokens] = v[p].to(dtype)
    table = torch.zeros(3, n_seq_pages, dtype=torch.int32)
    table[1] = perm.to(torch.int32)
    return kp, vp, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window,cap,splits", [
    (4, 2, 16, 0, 0.0, 1), (3, 1, 48, 7, 20.0, 3), (8, 4, 256, 40, 50.0, 5),
    (2, 2, 128, 0, 0.0, 16), (6, 3, 512, 33, 0.0, 2)])
def test_attention_rows_over_cache_and_fresh(dtype, nh, nkv, hd, window, cap, splits):
    """Single rows deep in a sequence read the paged cache (with a ring when
    there is a window); whole prompts read the step's own rows."""
    n = _native()
    g = torch.Generator().manual_seed(3)
    T = 150
    q = torch.randn(T, nh, hd, generator=g).to(dtype)
    k = torch.randn(T, nkv, hd, generator=g).to(dtype)
    v = torch.randn(T, nkv, hd, generator=g).to(dtype)
    scale = 3.0 / math.sqrt(hd)
    ref = plain.attention(q.double(), k.double(), v.double(), scale, cap, window)
    page = 8
    ring = (-(-window // page) + 1) * page if window else 0
    # (a) the last rows, one per launch-row, from the cache
    rows = [T - 1, T - 2, 60, 5, 0]
    for r in rows:
        keep = range(max(0, r + 1 - ring), r + 1) if ring else range(r + 1)
        kp, vp, table = _paged(k, v, page, ring, nkv, hd, dtype, keep)
        out = torch.empty(1, nh * hd, dtype=dtype, device=DEV)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
        scratch = torch.empty(max(1, n.attention_rows_scratch_bytes(1, nh, hd, splits)),
                              dtype=torch.uint8, device=DEV)
        qr = q[r].reshape(1, nh * hd).contiguous().to(DEV)
        n.attention_rows(qr, nh * hd, None, None, nh * hd, kp.to(DEV), vp.to(DEV), table.to(DEV),
                         page, ring, i32([r]), i32([0]), i32([1]), i32([r]), i32([0]), out,
                         scratch, nh, nkv, hd, scale, cap, window, splits)
        _close(out.view(nh, hd), ref[r], dtype, f"cache row {r}", factor=4)
    # (b) two packed prompts (the sequence and its first 21 tokens) from fresh rows
    T2 = 21
    packed = torch.cat([torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1),
                        torch.cat([q[:T2].reshape(T2, -1), k[:T2].reshape(T2, -1),
                                   v[:T2].reshape(T2, -1)], dim=1)], dim=0).contiguous().to(DEV)
    width = (nh + 2 * nkv) * hd
    out = torch.empty(T + T2, nh * hd, dtype=dtype, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    n.attention_rows(packed, width, packed[:, nh * hd:], packed[:, (nh + nkv) * hd:], width,
                     None, None, None, page, ring,
                     i32(list(range(T)) + list(range(T2))), i32([0] * T + [1] * T2), i32([0, 2]),
                     i32([0, 0]), i32([0, T]), out, None, nh, nkv, hd, scale, cap, window, 1)
    _close(out[:T].view(T, nh, hd), ref, dtype, "fresh rows, sequence 0", factor=4)
    _close(out[T:].view(T2, nh, hd), ref[:T2], dtype, "fresh rows, sequence 1", factor=4)


@pytest.mark.parametrize("nh,nkv,hd,window,cap,splits,warps", [
    (4, 2, 64, 0, 0.0, 1, 4), (8, 4, 256, 40, 50.0, 5, 4), (8, 1, 128, 0, 30.0, 3, 2),
    (2, 2, 128, 21, 0.0, 16, 1), (8, 4, 256, 0, 0.0, 2, 1), (4, 1, 256, 100, 50.0, 1, 2),
    (8, 4, 256, 0, 50.0, 1, 1), (16, 2, 64, 0, 0.0, 7, 4),
    # blocks of 8 warps: a thread per pair of output columns (accumulators asked for ahead of
    # the maxima) and fewer threads than that; more runs than are asked for ahead; one run
    (8, 4, 256, 0, 50.0, 4, 8), (8, 4, 256, 40, 50.0, 2, 8), (16, 2, 64, 0, 0.0, 3, 8),
    (4, 2, 128, 0, 30.0, 40, 8), (2, 2, 128, 21, 0.0, 1, 8), (8, 1, 256, 0, 0.0, 2, 8),
    # the ways the runs are joined: by a warp for its own columns (one or two pairs of columns
    # a thread; up to 16, 32 or 64 runs) and by the whole block (more runs or more columns)
    (2, 2, 256, 0, 0.0, 20, 4), (8, 4, 256, 0, 50.0, 20, 4), (2, 2, 256, 30, 0.0, 40, 4),
    (8, 2, 256, 0, 0.0, 5, 8), (16, 2, 128, 25, 30.0, 3, 8), (8, 4, 256, 0, 0.0, 70, 8)])
def test_attention_decode_kernel(nh, nkv, hd, window, cap, splits, warps):
    """The bfloat16 decode kernel: rows at tile and page edges, with and
    without a ring, several rows of different sequences in one launch."""
    n = _native()
    assert n.attention_decode_supports(nh, nkv, hd, 16)
    assert not n.attention_decode_supports(nh, nkv, 48, 16)
    assert not n.attention_decode_supports(nh, nkv, hd, 8)
    g = torch.Generator().manual_seed(13)
    T = 150
    dtype = torch.bfloat16
    q = torch.randn(T, nh, hd, generator=g).to(dtype)
    k = torch.randn(T, nkv, hd, generator=g).to(dtype)
    v = torch.randn(T, nkv, hd, generator=g).to(dtype)
    scale = 3.0 / math.sqrt(hd)
    ref = plain.attention(q.double(), k.double(), v.double(), scale, cap, window)
    page = 16
    ring = (-(-window // page) + 1) * page if window else 0
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    rows = [T - 1, 100, 64, 63, 48, 47, 33, 32, 31, 17, 16, 15, 1, 0]
    tickets = torch.zeros(3 * nkv, dtype=torch.int32, device=DEV)
    for r in rows:
        keep = range(max(0, r + 1 - ring), r + 1) if ring else range(r + 1)
        kp, vp, table = _paged(k, v, page, ring, nkv, hd, dtype, keep)
        kp, vp = torch.nan_to_num(kp, nan=1e4), torch.nan_to_num(vp, nan=1e4)   # loud if read
        out = torch.empty(1, nh * hd, dtype=dtype, device=DEV)
        scratch = torch.empty(max(1, n.attention_rows_scratch_bytes(1, nh, hd, splits)),
                              dtype=torch.uint8, device=DEV)
        qr = q[r].reshape(1, nh * hd).contiguous().to(DEV)
        n.attention_decode(qr, nh * hd, kp.to(DEV), vp.to(DEV), table.to(DEV), page, ring,
                           i32([r]), i32([0]), i32([1]), out, scratch, tickets, nh, nkv, hd, scale,
                           cap, window, splits, warps)
        assert int(tickets.abs().sum()) == 0, "the ticket counters are put back"
        _close(out.view(nh, hd), ref[r], dtype, f"decode row {r}")
    # several rows in one launch: rows of two sequences (slots 1 and 2 hold the same pages)
    if not ring:
        kp, vp, table = _paged(k, v, page, 0, nkv, hd, dtype, range(T))
        table[2] = table[1]
        picks = [T - 1, 77, 5]
        qs = torch.stack([q[r].reshape(nh * hd) for r in picks]).contiguous().to(DEV)
        out = torch.empty(3, nh * hd, dtype=dtype, device=DEV)
        scratch = torch.empty(max(1, n.attention_rows_scratch_bytes(3, nh, hd, splits)),
                              dtype=torch.uint8, device=DEV)
        n.attention_decode(qs, nh * hd, kp.to(DEV), vp.to(DEV), table.to(DEV), page, 0,
                           i32(picks), i32([0, 1, 1]), i32([1, 2]), out, scratch, tickets, nh, nkv,
                           hd, scale, cap, window, splits, warps)
        for i, r in enumerate(picks):
            _close(out[i].view(nh, hd), ref[r], dtype, f"decode rows together, row {r}")


@pytest.mark.parametrize("nh,nkv,hd,window,cap", [
    (4, 2, 64, 0, 0.0), (8, 4, 256, 100, 50.0), (4, 1, 128, 0, 30.0), (2, 2, 128, 70, 0.0),
    (8, 4, 256, 0, 0.0), (3, 3, 64, 17, 20.0)])
def test_attention_prefill_kernel(nh, nkv, hd, window, cap):
    """The bfloat16 prompt kernel on packed prompts of unequal lengths (one
    shorter than a tile, one that ends inside a tile, one of whole tiles)."""
    n = _native()
    assert n.attention_prefill_supports(nh, nkv, hd)
    assert not n.attention_prefill_supports(8, 1, hd) and not n.attention_prefill_supports(nh, nkv, 48)
    g = torch.Generator().manual_seed(14)
    lens = [200, 5, 64, 131]
    dtype = torch.bfloat16
    scale = 3.0 / math.sqrt(hd)
    qs, ks, vs, refs = [], [], [], []
    for T in lens:
        q = torch.randn(T, nh, hd, generator=g).to(dtype)
        k = torch.randn(T, nkv, hd, generator=g).to(dtype)
        v = torch.randn(T, nkv, hd, generator=g).to(dtype)
        refs.append(plain.attention(q.double(), k.double(), v.double(), scale, cap, window))
        qs.append(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
    packed = torch.cat(qs, dim=0).contiguous().to(DEV)
    out = torch.full((sum(lens), nh * hd), float("nan"), dtype=dtype, device=DEV)
    row0 = [0]
    for T in lens[:-1]:
        row0.append(row0[-1] + T)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    n.attention_prefill(packed, out, i32(row0), i32(lens), len(lens), max(lens), nh, nkv, hd,
                        scale, cap, window)
    for r0, T, ref in zip(row0, lens, refs):
        _close(out[r0:r0 + T].view(T, nh, hd), ref, dtype, f"prefill, sequence of {T}")


@pytest.mark.parametrize("nh,nkv,hd,window,cap,boost", [
    (4, 2, 64, 0, 0.0, 1.0), (8, 4, 256, 100, 50.0, 1.0), (2, 2, 128, 70, 0.0, 1.0),
    (8, 4, 256, 0, 0.0, 1.0), (3, 3, 64, 17, 20.0, 1.0), (4, 2, 128, 0, 30.0, 1.0),
    (8, 4, 256, 0, 50.0, 6.0), (4, 2, 128, 150, 10.0, 3.0)])
def test_attention_prefill_tc_kernel(nh, nkv, hd, window, cap, boost):
    """The tcgen05 prompt kernel on packed prompts of unequal lengths.  `boost` makes the
    scores large against the cap, where the kernel takes the tanh from the
    special-function unit instead of the short series it uses for small arguments."""
    n = _native()
    assert n.attention_prefill_tc_supports(nh, nkv, hd, (nh + 2 * nkv) * hd)
    assert not n.attention_prefill_tc_supports(8, 2, hd, 12 * hd)
    g = torch.Generator().manual_seed(15)
    lens = [200, 5, 64, 131, 300]
    dtype = torch.bfloat16
    scale = 3.0 * boost / math.sqrt(hd)
    qs, refs = [], []
    for T in lens:
        q = torch.randn(T, nh, hd, generator=g).to(dtype)
        k = torch.randn(T, nkv, hd, generator=g).to(dtype)
        v = torch.randn(T, nkv, hd, generator=g).to(dtype)
        refs.append(plain.attention(q.double(), k.double(), v.double(), scale, cap, window))
        qs.append(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
    packed = torch.cat(qs, dim=0).contiguous().to(DEV)
    out = torch.full((sum(lens), nh * hd), float("nan"), dtype=dtype, device=DEV)
    row0 = [0]
    for T in lens[:-1]:
        row0.append(row0[-1] + T)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    n.attention_prefill_tc(packed, out, i32(row0), i32(lens), len(lens), max(lens), nh, nkv, hd,
                           scale, cap, window)
    assert n.attention_prefill_tc_error() == 0
    for r0, T, ref in zip(row0, lens, refs):
        _close(out[r0:r0 + T].view(T, nh, hd), ref, dtype, f"tcgen05 prefill, sequence of {T}")


@pytest.mark.parametrize("nh,nkv,hd,window,cap", [
    (4, 2, 256, 0, 50.0), (2, 2, 128, 0, 0.0), (4, 2, 128, 900, 30.0), (2, 1, 64, 0, 0.0)])
def test_attention_prefill_tc_kernel_splits_long_blocks(nh, nkv, hd, window, cap):
    """Few blocks of query rows: those with many key tiles are run as two halves whose
    partial results the later one joins; twice in a row through the same tickets."""
    n = _native()
    g = torch.Generator().manual_seed(16)
    lens = [1100, 70]                      # few enough blocks to fill half of the device at most
    dtype = torch.bfloat16
    scale = 3.0 / math.sqrt(hd)
    qs, refs = [], []
    for T in lens:
        q = torch.randn(T, nh, hd, generator=g).to(dtype)
        k = torch.randn(T, nkv, hd, generator=g).to(dtype)
        v = torch.randn(T, nkv, hd, generator=g).to(dtype)
        refs.append(plain.attention(q.double(), k.double(), v.double(), scale, cap, window))
        qs.append(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
    packed = torch.cat(qs, dim=0).contiguous().to(DEV)
    row0 = [0, lens[0]]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    need, n_tickets = n.attention_prefill_tc_split(len(lens), max(lens), nh, nkv, hd)
    if os.environ.get("SIB_PREFILL_SPLIT") == "0":
        pytest.skip("the split is switched off")
    assert need > 0 and n_tickets > 0, "a launch this small splits"
    scratch = torch.empty(need, dtype=torch.uint8, device=DEV)
    tickets = torch.zeros(n_tickets, dtype=torch.int32, device=DEV)
    for call in range(2):
        out = torch.full((sum(lens), nh * hd), float("nan"), dtype=dtype, device=DEV)
        n.attention_prefill_tc(packed, out, i32(row0), i32(lens), len(lens), max(lens), nh, nkv, hd,
                               scale, cap, window, scratch, tickets)
        assert n.attention_prefill_tc_error() == 0
        assert int(tickets.abs().sum()) == 0, "the tickets are put back"
        for r0, T, ref in zip(row0, lens, refs):
            _close(out[r0:r0 + T].view(T, nh, hd), ref, dtype, f"split prefill, sequence of {T}, call {call}")


@pytest.mark.parametrize("nh,nkv,hd,window,cap,lens", [
    (8, 4, 256, 0, 50.0, [2048]), (4, 2, 256, 700, 50.0, [1500, 40, 333]),
    (2, 2, 128, 0, 0.0, [900, 1100]), (2, 1, 64, 0, 0.0, [1300, 129, 5]),
    (4, 2, 128, 300, 30.0, [64, 2000]), (8, 4, 256, 0, 0.0, [300])])
def test_attention_prefill_tc_kernel_as_a_balanced_list_of_work(nh, nkv, hd, window, cap, lens):
    """With the prompts' lengths known on the host the launch is a list of work items, the
    longest first, and the blocks are split whose halves make the busiest SM's share
    smallest: the same results as the plain implementation, twice through the same
    tickets; without memory for the split blocks it falls back to a grid."""
    n = _native()
    g = torch.Generator().manual_seed(17)
    dtype = torch.bfloat16
    scale = 3.0 / math.sqrt(hd)
    qs, refs = [], []
    for T in lens:
        q = torch.randn(T, nh, hd, generator=g).to(dtype)
        k = torch.randn(T, nkv, hd, generator=g).to(dtype)
        v = torch.randn(T, nkv, hd, generator=g).to(dtype)
        refs.append(plain.attention(q.double(), k.double(), v.double(), scale, cap, window))
        qs.append(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
    packed = torch.cat(qs, dim=0).contiguous().to(DEV)
    row0 = [0]
    for T in lens[:-1]:
        row0.append(row0[-1] + T)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    n_items, need, n_tickets = n.attention_prefill_tc_plan(lens, nh, nkv, hd, window)
    if os.environ.get("SIB_PREFILL_BALANCE") == "0":
        pytest.skip("the balanced list is switched off")
    span = 128 // (nh // nkv) * (2 if hd >= 128 else 1)
    blocks = sum(-(-T // span) for T in lens) * nkv
    assert n_items >= blocks                      # every block once, split ones twice
    assert (n_items > blocks) == (need > 0)
    if max(lens) >= 1000:
        assert need > 0, "a long prompt alone on the device has blocks worth splitting"
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    tickets = torch.zeros(max(n_tickets, 1), dtype=torch.int32, device=DEV)
    for call in range(3):
        out = torch.full((sum(lens), nh * hd), float("nan"), dtype=dtype, device=DEV)
        # (the third call brings no memory: a grid, unless nothing was to be split anyway)
        mem = (scratch, tickets) if call < 2 else (None, None)
        n.attention_prefill_tc(packed, out, i32(row0), i32(lens), len(lens), max(lens), nh, nkv, hd,
                               scale, cap, window, mem[0], mem[1], lens)
        assert n.attention_prefill_tc_error() == 0
        assert int(tickets.abs().sum()) == 0, "the tickets are put back"
        for r0, T, ref in zip(row0, lens, refs):
            _close(out[r0:r0 + T].view(T, nh, hd), ref, dtype, f"balanced prefill, sequence of {T}, call {call}")


@pytest.mark.parametrize("nh,nkv,hd,window,lens,q0s", [
    (8, 4, 256, 0, [1500], [1300]), (4, 2, 128, 200, [900, 333], [700, 332]),
    (2, 2, 64, 0, [700, 64, 300], [650, 0, 129]), (4, 2, 256, 96, [200, 51], [168, 50])])
def test_attention_prefill_tc_kernel_with_rows_that_are_keys_only(nh, nkv, hd, window, lens, q0s):
    """The rows of a sequence before its first query position bring keys and values only:
    the later rows' results are the plain implementation's over the whole sequence, the
    earlier rows of the output are not written; as a balanced list and as a grid.  The q
    columns of the earlier rows hold NaN, which must not reach any result."""
    n = _native()
    g = torch.Generator().manual_seed(19)
    dtype = torch.bfloat16
    scale = 3.0 / math.sqrt(hd)
    qs, refs = [], []
    for T, q0 in zip(lens, q0s):
        q = torch.randn(T, nh, hd, generator=g).to(dtype)
        k = torch.randn(T, nkv, hd, generator=g).to(dtype)
        v = torch.randn(T, nkv, hd, generator=g).to(dtype)
        refs.append(plain.attention(q.double(), k.double(), v.double(), scale, 30.0, window))
        q = q.clone()
        q[:q0] = float("nan")
        qs.append(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
    packed = torch.cat(qs, dim=0).contiguous().to(DEV)
    row0 = [0]
    for T in lens[:-1]:
        row0.append(row0[-1] + T)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    n_items, need, n_tickets = n.attention_prefill_tc_plan(lens, nh, nkv, hd, window, q0s)
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    tickets = torch.zeros(max(n_tickets, 1), dtype=torch.int32, device=DEV)
    for host in (lens, None):
        out = torch.full((sum(lens), nh * hd), float("nan"), dtype=dtype, device=DEV)
        n.attention_prefill_tc(packed, out, i32(row0), i32(lens), len(lens), max(lens), nh, nkv, hd,
                               scale, 30.0, window, scratch, tickets, host, i32(q0s),
                               q0s if host else None)
        assert n.attention_prefill_tc_error() == 0
        for r0, T, q0, ref in zip(row0, lens, q0s, refs):
            _close(out[r0 + q0:r0 + T].view(T - q0, nh, hd), ref[q0:], dtype,
                   f"rows from {q0} of a sequence of {T}")
            assert torch.isnan(out[r0:r0 + q0].float()).all(), "rows that are keys only were written"


def test_gather_kv_rows_brings_pages_back_into_packed_rows():
    n = _native()
    g = torch.Generator().manual_seed(20)
    nh, nkv, hd, page, ring = 3, 2, 16, 4, 12
    n_pages, slots, max_pages = 40, 3, 10
    k_pool = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16).to(DEV)
    v_pool = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16).to(DEV)
    table = torch.randperm(n_pages, generator=g)[:slots * max_pages].view(slots, max_pages).to(torch.int32).to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    seq_slot, first, upto, row0 = [2, 0], [3, 20], [17, 29], [0, 17]
    width = (nh + 2 * nkv) * hd
    for ring_tokens in (0, ring):
        packed = torch.full((17 + 29, width), 7.0, dtype=torch.bfloat16, device=DEV)
        n.gather_kv_rows(packed, k_pool, v_pool, table, i32(seq_slot), i32(first), i32(upto), i32(row0),
                         14, page, ring_tokens, nh, nkv, hd)
        got = packed.cpu()
        for b in range(2):
            for pos in range(0 if b == 0 else 0, upto[b]):
                row = got[row0[b] + pos]
                if pos < first[b]:
                    assert (row == 7.0).all(), "a position that was not asked for was written"
                    continue
                cell = pos % ring_tokens if ring_tokens else pos
                pg = int(table[seq_slot[b], cell // page])
                assert (row[:nh * hd] == 0).all()
                want_k = k_pool[pg, :, cell % page].reshape(-1).cpu()
                want_v = v_pool[pg, :, cell % page].reshape(-1).cpu()
                assert torch.equal(row[nh * hd:(nh + nkv) * hd], want_k)
                assert torch.equal(row[(nh + nkv) * hd:], want_v)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("style", [0, 1])
@pytest.mark.parametrize("hd,rot", [(48, 32), (64, 64), (16, 16)])
def test_rope_store(dtype, style, hd, rot):
    n = _native()
    g = torch.Generator().manual_seed(4)
    nh, nkv = 3, 2
    theta = 777.0
    positions = [0, 1, 2, 3, 4, 17, 18, 19, 20]        # two sequences: 5 rows from 0, 4 rows from 17
    R = len(positions)
    qkv = torch.randn(R, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    page, ring = 4, 8
    kp = torch.zeros(9, nkv, page, hd, dtype=dtype, device=DEV)
    vp = torch.zeros(9, nkv, page, hd, dtype=dtype, device=DEV)
    table = torch.tensor([[3, 5], [0, 0], [7, 2]], dtype=torch.int32, device=DEV)
    inv_freq = torch.pow(torch.tensor(theta), (-1.0 / rot) * torch.arange(rot // 2).float() * 2)
    buf = qkv.clone().to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    n.rope_store(buf, i32(positions), i32([0] * 5 + [1] * 4), i32([2, 0]), i32([5, 21]),
                 inv_freq.to(DEV), rot, style, kp, vp, table, page, ring, nh, nkv, hd)

    def rot_ref(x):  # x [R, heads, hd]
        x = x.double()
        ang = torch.tensor(positions).double()[:, None] * inv_freq.double()[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = x.clone()
        if style == 0:
            a, b = x[..., :rot // 2], x[..., rot // 2:rot]
            out[..., :rot // 2], out[..., rot // 2:rot] = a * c - b * s, a * s + b * c
        else:
            a, b = x[..., 0:rot:2], x[..., 1:rot:2]
            out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s, a * s + b * c
        return out
    qd = qkv.double()
    q_ref = rot_ref(qd[:, :nh * hd].view(R, nh, hd))
    k_ref = rot_ref(qd[:, nh * hd:(nh + nkv) * hd].view(R, nkv, hd))
    v_ref = qd[:, (nh + nkv) * hd:].view(R, nkv, hd)
    got = buf.double().cpu()
    _close(got[:, :nh * hd].view(R, nh, hd), q_ref, dtype, "q rotated in place")
    _close(got[:, nh * hd:(nh + nkv) * hd].view(R, nkv, hd), k_ref, dtype, "k rotated in place")
    # cache cells: sequence 0 -> slot 2 (pages 7, 2), sequence 1 -> slot 0 (pages 3, 5)
    tab = table.cpu()
    for r, p in enumerate(positions):
        slot = 2 if r < 5 else 0
        cell = p % ring
        pg = int(tab[slot, cell // page])
        _close(kp[pg, :, cell % page].cpu(), k_ref[r], dtype, f"k cell of row {r}")
        _close(vp[pg, :, cell % page].cpu(), v_ref[r], dtype, f"v cell of row {r}")


@pytest.mark.parametrize("hd,nh,nkv,K", [(32, 3, 2, 72), (256, 8, 4, 256), (64, 2, 1, 40), (16, 4, 0, 64)])
def test_skinny_linear_that_rotates_and_stores(hd, nh, nkv, K):
    """The q|k|v product of a few rows with rotation and cache write in its epilogue: the rows
    of two sequences, one of them in a ring; nkv = 0 projects q only and stores nothing."""
    n = _native()
    g = torch.Generator().manual_seed(40 + hd)
    theta = 500.0
    positions = [0, 1, 2, 3, 4, 17, 18, 19, 20]
    R = len(positions)
    N = (nh + 2 * nkv) * hd
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    page, ring = 4, 8
    kp = torch.zeros(9, max(nkv, 1), page, hd, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    table = torch.tensor([[3, 5], [0, 0], [7, 2]], dtype=torch.int32, device=DEV)
    inv_freq = torch.pow(torch.tensor(theta), (-1.0 / hd) * torch.arange(hd // 2).float() * 2)
    out = torch.full((R, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    n.skinny_linear_rope(x.to(DEV), w.to(DEV), out, i32(positions), i32([0] * 5 + [1] * 4),
                         i32([2, 0]), i32([5, 21]), inv_freq.to(DEV), kp if nkv else None,
                         vp if nkv else None, table if nkv else None, page, ring, nh, nkv, hd)
    y = x.double() @ w.double().T

    def rot_ref(v):  # v [R, heads, hd]
        ang = torch.tensor(positions).double()[:, None] * inv_freq.double()[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat([a * c - b * s, a * s + b * c], dim=-1)
    q_ref = rot_ref(y[:, :nh * hd].view(R, nh, hd))
    got = out.double().cpu()
    _close(got[:, :nh * hd].view(R, nh, hd), q_ref, torch.bfloat16, "q rotated")
    if not nkv:
        return
    k_ref = rot_ref(y[:, nh * hd:(nh + nkv) * hd].view(R, nkv, hd))
    v_ref = y[:, (nh + nkv) * hd:].view(R, nkv, hd)
    _close(got[:, nh * hd:(nh + nkv) * hd].view(R, nkv, hd), k_ref, torch.bfloat16, "k rotated")
    _close(got[:, (nh + nkv) * hd:].view(R, nkv, hd), v_ref, torch.bfloat16, "v")
    tab = table.cpu()
    for r, pos in enumerate(positions):
        slot = 2 if r < 5 else 0
        cell = pos % ring
        pg = int(tab[slot, cell // page])
        _close(kp[pg, :, cell % page].cpu(), k_ref[r], torch.bfloat16, f"k cell of row {r}")
        _close(vp[pg, :, cell % page].cpu(), v_ref[r], torch.bfloat16, f"v cell of row {r}")


def test_rope_store_ring_keeps_only_the_last_positions():
    """A prompt longer than the ring: only its last ring_tokens positions are written."""
    n = _native()
    nh, nkv, hd = 1, 1, 16
    T, page, ring = 20, 4, 8
    qkv = torch.arange(T, dtype=torch.float32).repeat_interleave(3 * hd).view(T, 3 * hd).to(DEV)
    kp = torch.full((2, nkv, page, hd), -1.0, device=DEV)
    vp = torch.full((2, nkv, page, hd), -1.0, device=DEV)
    table = torch.tensor([[1, 0]], dtype=torch.int32, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    n.rope_store(qkv, i32(list(range(T))), i32([0] * T), i32([0]), i32([T]), None, 0, 0,
                 kp, vp, table, page, ring, nh, nkv, hd)
    for p in range(T - ring, T):
        cell = p % ring
        pg = [1, 0][cell // page]
        assert float(vp[pg, 0, cell % page, 0]) == float(p)


@pytest.mark.parametrize("R", [1, 3, 8, 13, 32, 64])
@pytest.mark.parametrize("N,K", [(48, 64), (300, 96), (2304, 2048), (1000, 200)])
def test_skinny_linear(R, N, K):
    n = _native()
    g = torch.Generator().manual_seed(5)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    out = torch.empty(R, N, dtype=torch.float32, device=DEV)
    n.skinny_linear(x.to(DEV), w.to(DEV), out)
    _close(out, ref, torch.float32, "skinny f32 out", factor=20)
    out16 = torch.empty(R, N, dtype=torch.bfloat16, device=DEV)
    n.skinny_linear(x.to(DEV), w.to(DEV), out16)
    _close(out16, ref, torch.bfloat16, "skinny bf16 out")
    capped = torch.empty(R, N, dtype=torch.float32, device=DEV)
    n.skinny_linear(x.to(DEV), w.to(DEV), capped, n.EPI_SOFTCAP, 0.7)
    _close(capped, 0.7 * torch.tanh(ref / 0.7), torch.float32, "skinny soft cap", factor=20)
    if N % 16 == 0:
        gated = torch.empty(R, N // 2, dtype=torch.bfloat16, device=DEV)
        n.skinny_linear(x.to(DEV), w.to(DEV), gated, n.EPI_GEGLU)
        y = ref.view(R, N // 16, 2, 8)
        _close(gated, (plain.gelu_tanh(y[:, :, 0]) * y[:, :, 1]).reshape(R, N // 2),
               torch.bfloat16, "skinny gated")


@pytest.mark.parametrize("R,N,K,ksplit,stages", [
    (1, 128, 64, 0, 0), (3, 144, 200, 0, 0), (8, 2304, 2048, 0, 0), (16, 4096, 2304, 0, 0),
    (9, 300, 328, 1, 2), (16, 272, 1024, 8, 2), (5, 48, 1600, 5, 3), (12, 1000, 776, 3, 12),
    (2, 18432, 2304, 0, 0), (7, 2304, 9216, 0, 0), (1, 256, 128, 2, 1),
])
def test_linear_stream(R, N, K, ksplit, stages):
    """The few-row product with TMA-staged weights: sizes that are no multiples of its
    tiles (rows of 128, k of 64), every split of k over a cluster, rings shorter and longer
    than the run of k, all epilogues and both output types."""
    n = _native()
    g = torch.Generator().manual_seed(6)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    xd, wd = x.to(DEV), w.to(DEV)
    out = torch.full((R, N), float("nan"), dtype=torch.float32, device=DEV)
    n.linear_stream(xd, wd, out, n.EPI_NONE, 0.0, ksplit, stages)
    _close(out, ref, torch.float32, "stream f32 out", factor=20)
    # a strided input (rows of a wider buffer) and a strided output
    wide = torch.zeros(R, K + 16, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = xd
    out16 = torch.full((R, N + 8), float("nan"), dtype=torch.bfloat16, device=DEV)
    n.linear_stream(wide[:, :K], wd, out16[:, :N], n.EPI_NONE, 0.0, ksplit, stages)
    _close(out16[:, :N], ref, torch.bfloat16, "stream bf16 out")
    assert torch.isnan(out16[:, N:].float()).all()
    capped = torch.empty(R, N, dtype=torch.float32, device=DEV)
    n.linear_stream(xd, wd, capped, n.EPI_SOFTCAP, 0.7, ksplit, stages)
    _close(capped, 0.7 * torch.tanh(ref / 0.7), torch.float32, "stream soft cap", factor=20)
    if N % 16 == 0:
        gated = torch.empty(R, N // 2, dtype=torch.bfloat16, device=DEV)
        n.linear_stream(xd, wd, gated, n.EPI_GEGLU, 0.0, ksplit, stages)
        y = ref.view(R, N // 16, 2, 8)
        _close(gated, (plain.gelu_tanh(y[:, :, 0]) * y[:, :, 1]).reshape(R, N // 2),
               torch.bfloat16, "stream gated")
    # the same sums whatever the split and the ring (up to the order of the partial sums)
    again = torch.empty(R, N, dtype=torch.float32, device=DEV)
    n.linear_stream(xd, wd, again, n.EPI_NONE, 0.0, 1, 2)
    _close(again, out.double().cpu(), torch.float32, "stream, one block a tile", factor=5)
    torch.cuda.synchronize()
    watch = n.KernelWatch()
    watch.fetch()
    torch.cuda.synchronize()
    watch.check()


def test_linear_stream_refuses_what_it_cannot_do():
    n = _native()
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(n.KernelError, match="1 to 16 rows"):
        n.linear_stream(torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV), w,
                        torch.empty(17, 32, dtype=torch.float32, device=DEV))
    with pytest.raises(n.KernelError, match="multiples of 8"):
        n.linear_stream(torch.zeros(2, 60, dtype=torch.bfloat16, device=DEV),
                        torch.zeros(32, 60, dtype=torch.bfloat16, device=DEV),
                        torch.empty(2, 32, dtype=torch.float32, device=DEV))
    with pytest.raises(n.KernelError, match="groups of 16"):
        n.linear_stream(torch.zeros(2, 64, dtype=torch.bfloat16, device=DEV),
                        torch.zeros(24, 64, dtype=torch.bfloat16, device=DEV),
                        torch.empty(2, 12, dtype=torch.bfloat16, device=DEV), n.EPI_GEGLU)


@pytest.mark.parametrize("R,N,K,ksplit,stages", [
    (17, 256, 256, 0, 0), (64, 2304, 2048, 0, 0), (33, 144, 72, 1, 1), (128, 4096, 2304, 0, 0),
    (100, 300, 328, 2, 2), (48, 272, 1024, 8, 3), (21, 48, 1600, 4, 2), (96, 1000, 776, 8, 8),
    (64, 18432, 2304, 0, 0), (32, 2304, 9216, 0, 0), (1, 256, 128, 2, 1), (16, 640, 520, 4, 0),
])
def test_linear_rows_tc(R, N, K, ksplit, stages):
    """The weight-streaming product of up to 128 rows on tcgen05: sizes that are no multiples
    of its tiles (128 weight rows, 64 of k, 16 rows), every split of k over a cluster, rings
    shorter and longer than the run of k, all epilogues, both output types, strided rows."""
    n = _native()
    g = torch.Generator().manual_seed(7)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    # one entry far from the rest: a row or a run of k that is dropped or taken twice shows
    x[R - 1, K - 1] = 40.0
    w[N - 1, K - 1] = 3.0
    ref = x.double() @ w.double().T
    xd, wd = x.to(DEV), w.to(DEV)
    out = torch.full((R, N), float("nan"), dtype=torch.float32, device=DEV)
    n.linear_rows_tc(xd, wd, out, n.EPI_NONE, 0.0, ksplit, stages)
    _close(out, ref, torch.float32, "rows_tc f32 out", factor=20)
    wide = torch.zeros(R, K + 16, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = xd
    out16 = torch.full((R, N + 8), float("nan"), dtype=torch.bfloat16, device=DEV)
    n.linear_rows_tc(wide[:, :K], wd, out16[:, :N], n.EPI_NONE, 0.0, ksplit, stages)
    _close(out16[:, :N], ref, torch.bfloat16, "rows_tc bf16 out")
    assert torch.isnan(out16[:, N:].float()).all()
    capped = torch.empty(R, N, dtype=torch.float32, device=DEV)
    n.linear_rows_tc(xd, wd, capped, n.EPI_SOFTCAP, 0.7, ksplit, stages)
    _close(capped, 0.7 * torch.tanh(ref / 0.7), torch.float32, "rows_tc soft cap", factor=20)
    if N % 16 == 0:
        gated = torch.full((R, N // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
        n.linear_rows_tc(xd, wd, gated, n.EPI_GEGLU, 0.0, ksplit, stages)
        y = ref.view(R, N // 16, 2, 8)
        _close(gated, (plain.gelu_tanh(y[:, :, 0]) * y[:, :, 1]).reshape(R, N // 2),
               torch.bfloat16, "rows_tc gated")
    again = torch.empty(R, N, dtype=torch.float32, device=DEV)
    n.linear_rows_tc(xd, wd, again, n.EPI_NONE, 0.0, 1, 2)
    _close(again, out.double().cpu(), torch.float32, "rows_tc, one block a tile", factor=5)
    torch.cuda.synchronize()
    watch = n.KernelWatch()
    watch.fetch()
    torch.cuda.synchronize()
    watch.check()


def test_linear_rows_tc_refuses_what_it_cannot_do():
    n = _native()
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(n.KernelError, match="1 to 128"):
        n.linear_rows_tc(torch.zeros(129, 64, dtype=torch.bfloat16, device=DEV), w,
                         torch.empty(129, 32, dtype=torch.float32, device=DEV))
    with pytest.raises(n.KernelError, match="multiples of 8"):
        n.linear_rows_tc(torch.zeros(20, 60, dtype=torch.bfloat16, device=DEV),
                         torch.zeros(32, 60, dtype=torch.bfloat16, device=DEV),
                         torch.empty(20, 32, dtype=torch.float32, device=DEV))
    with pytest.raises(n.KernelError, match="groups of 16"):
        n.linear_rows_tc(torch.zeros(20, 64, dtype=torch.bfloat16, device=DEV),
                         torch.zeros(24, 64, dtype=torch.bfloat16, device=DEV),
                         torch.empty(20, 12, dtype=torch.bfloat16, device=DEV), n.EPI_GEGLU)


def _chain_case(R, H, nh, nkv, hd, inter, seed):
    """Operands of a decoder's steps between two attention kernels, for R rows."""
    g = torch.Generator().manual_seed(seed)
    bf = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).to(DEV)  # noqa: E731
    f32 = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(DEV)  # noqa: E731
    return dict(
        attn=bf(R, nh * hd), w_o=bf(H, nh * hd, s=(nh * hd) ** -0.5), h=f32(R, H),
        g_post=f32(H, s=0.3) + 1, g_pre=f32(H, s=0.3) + 1, g_post2=f32(H, s=0.3) + 1,
        g_next=f32(H, s=0.3) + 1, w_gu=bf(2 * inter, H, s=H ** -0.5), w_down=bf(H, inter, s=inter ** -0.5),
        w_qkv=bf((nh + 2 * nkv) * hd, H, s=H ** -0.5))


@pytest.mark.parametrize("R,H,nh,nkv,hd,inter", [
    (3, 320, 4, 2, 32, 400), (8, 2304, 8, 4, 256, 9216), (13, 200, 5, 1, 48, 104),
    (16, 1024, 6, 3, 128, 1200), (1, 64, 4, 2, 16, 128),
])
def test_decode_chain_runs_a_layers_steps_as_one_kernel(R, H, nh, nkv, hd, inter):
    """Output projection, norm-add-norm, gated feed-forward, norm-add-norm and the next
    q|k|v with rotation and cache write as ONE kernel, against the same steps run one
    kernel each and against the plain implementation's functions."""
    n = _native()
    c = _chain_case(R, H, nh, nkv, hd, inter, seed=R + H)
    eps1, eps2 = 1e-6, 1e-5
    theta, page, ring = 700.0, 8, 0
    positions = [5 + 3 * i for i in range(R)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    row_pos, row_seq, seq_slot = i32(positions), i32(list(range(R))), i32(list(range(R)))
    seq_end = i32([p + 1 for p in positions])
    pages_per_seq = -(-(max(positions) + 1) // page)
    table = torch.randperm(R * pages_per_seq).to(torch.int32).view(R, pages_per_seq).to(DEV)
    inv_freq = torch.pow(torch.tensor(theta), (-1.0 / hd) * torch.arange(hd // 2).float() * 2).to(DEV)
    N3 = (nh + 2 * nkv) * hd

    def pools():
        z = torch.zeros(R * pages_per_seq, nkv, page, hd, dtype=torch.bfloat16, device=DEV)
        return z, z.clone()

    # the steps one kernel each
    a1 = torch.empty(R, H, dtype=torch.bfloat16, device=DEV)
    n.skinny_linear(c["attn"], c["w_o"], a1)
    h1 = c["h"].clone()
    x1 = torch.empty(R, H, dtype=torch.bfloat16, device=DEV)
    n.add_rms_norm(a1, c["g_post"], eps1, h1, c["g_pre"], eps2, x1)
    t1 = torch.empty(R, inter, dtype=torch.bfloat16, device=DEV)
    n.skinny_linear(x1, c["w_gu"], t1, n.EPI_GEGLU)
    f1 = torch.empty(R, H, dtype=torch.bfloat16, device=DEV)
    n.skinny_linear(t1, c["w_down"], f1)
    x2 = torch.empty(R, H, dtype=torch.bfloat16, device=DEV)
    n.add_rms_norm(f1, c["g_post2"], eps1, h1, c["g_next"], eps2, x2)
    qkv1 = torch.empty(R, N3, dtype=torch.bfloat16, device=DEV)
    kp1, vp1 = pools()
    n.skinny_linear_rope(x2, c["w_qkv"], qkv1, row_pos, row_seq, seq_slot, seq_end, inv_freq,
                         kp1, vp1, table, page, ring, nh, nkv, hd)

    # the same as one kernel
    sync = torch.zeros(2, dtype=torch.int32, device=DEV)
    for stages in (0, 2):
        a2 = torch.full((R, H), float("nan"), dtype=torch.bfloat16, device=DEV)
        h2 = c["h"].clone()
        y1 = torch.full((R, H), float("nan"), dtype=torch.bfloat16, device=DEV)
        t2 = torch.full((R, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
        f2 = torch.full((R, H), float("nan"), dtype=torch.bfloat16, device=DEV)
        y2 = torch.full((R, H), float("nan"), dtype=torch.bfloat16, device=DEV)
        qkv2 = torch.full((R, N3), float("nan"), dtype=torch.bfloat16, device=DEV)
        kp2, vp2 = pools()
        rope = dict(row_pos=row_pos, row_seq=row_seq, seq_slot=seq_slot, seq_end=seq_end,
                    inv_freq=inv_freq, k_pool=kp2, v_pool=vp2, page_table=table, page_tokens=page,
                    ring_tokens=ring, n_heads=nh, n_kv=nkv, head_dim=hd)
        phases = [
            n.chain_product(c["attn"], c["w_o"], a2),
            n.chain_norm(a2, c["g_post"], eps1, h2, c["g_pre"], eps2, y1),
            n.chain_product(y1, c["w_gu"], t2, n.EPI_GEGLU),
            n.chain_product(t2, c["w_down"], f2),
            n.chain_norm(f2, c["g_post2"], eps1, h2, c["g_next"], eps2, y2),
            n.chain_product(y2, c["w_qkv"], qkv2, rope=rope),
        ]
        n.decode_chain(phases, R, sync, stages)
        torch.cuda.synchronize()
        assert sync.tolist() == [0, 0]                    # the counters were put back
        for got, want, what in ((a2, a1, "output projection"), (y1, x1, "first norm"),
                                (t2, t1, "gated product"), (f2, f1, "down"), (y2, x2, "second norm"),
                                (qkv2, qkv1, "q|k|v rotated"), (kp2, kp1, "keys in the cache"),
                                (vp2, vp1, "values in the cache")):
            assert torch.isfinite(got.float()).all(), what
            _close(got, want.double().cpu(), torch.bfloat16, f"chain, {what} (stages {stages})")
        # (the sub-layer outputs are bfloat16: one unit in their last place moves the sum)
        _close(h2, h1.double().cpu(), torch.bfloat16, "residual stream")
    # and against the plain functions (bfloat16 roundings of the intermediates apart)
    h0 = c["h"].double().cpu()
    a = c["attn"].double().cpu() @ c["w_o"].double().cpu().T
    r = h0 + plain.rms_norm(a, c["g_post"].double().cpu() - 1, eps1)
    x = plain.rms_norm(r, c["g_pre"].double().cpu() - 1, eps2)
    gu = (x @ c["w_gu"].double().cpu().T).view(R, inter // 8, 2, 8)
    t = (plain.gelu_tanh(gu[:, :, 0]) * gu[:, :, 1]).reshape(R, inter)
    f = t @ c["w_down"].double().cpu().T
    r2 = r + plain.rms_norm(f, c["g_post2"].double().cpu() - 1, eps1)
    _close(h2, r2, torch.bfloat16, "residual stream against plain")
    x_next = plain.rms_norm(r2, c["g_next"].double().cpu() - 1, eps2)
    q = (x_next @ c["w_qkv"].double().cpu().T)[:, :nh * hd].view(R, nh, hd)
    q_rot = torch.stack([plain.rope_neox(q[i:i + 1], torch.tensor([positions[i]]), theta)[0]
                         for i in range(R)])
    _close(qkv2[:, :nh * hd].view(R, nh, hd), q_rot, torch.bfloat16, "q against plain", factor=3)
    watch = n.KernelWatch()
    watch.fetch()
    torch.cuda.synchronize()
    watch.check()


def test_decode_chain_single_phases_and_refusals():
    n = _native()
    g = torch.Generator().manual_seed(3)
    sync = torch.zeros(2, dtype=torch.int32, device=DEV)
    for R, N, K in ((5, 1000, 328), (16, 256000, 256), (2, 48, 3072)):
        x = torch.randn(R, K, generator=g).to(torch.bfloat16).to(DEV)
        w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
        ref = x.double().cpu() @ w.double().cpu().T
        out = torch.full((R, N), float("nan"), dtype=torch.float32, device=DEV)
        n.decode_chain([n.chain_product(x, w, out, n.EPI_SOFTCAP, 0.9)], R, sync)
        _close(out, 0.9 * torch.tanh(ref / 0.9), torch.float32, f"capped 32-bit product {N}x{K}",
               factor=20)
    # a plain norm of chosen rows (what a model's last norm is)
    h = torch.randn(6, 200, generator=g).to(DEV)
    gain = (torch.randn(200, generator=g) * 0.2 + 1).to(DEV)
    rows = torch.tensor([4, 0, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(3, 200, dtype=torch.bfloat16, device=DEV)
    n.decode_chain([n.chain_norm(None, None, 0.0, h, gain, 1e-6, out, rows)], 3, sync)
    _close(out, plain.rms_norm(h[rows.long()].double().cpu(), gain.double().cpu() - 1, 1e-6),
           torch.bfloat16, "plain norm of chosen rows")
    x = torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(n.KernelError, match="1 to 16"):
        n.decode_chain([n.chain_product(x, w, torch.empty(17, 32, dtype=torch.bfloat16, device=DEV))],
                       17, sync)
    ph = n.chain_product(x[:2], w, torch.empty(2, 32, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(n.KernelError, match="phases"):
        n.decode_chain([ph] * 9, 2, sync)
    assert sync.tolist() == [0, 0]


def test_skinny_linear_refuses_what_it_cannot_do():
    n = _native()
    x = torch.zeros(65, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(16, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(n.KernelError, match="1 to 64"):
        n.skinny_linear(x, w, torch.empty(65, 16, dtype=torch.float32, device=DEV))
    x = torch.zeros(2, 60, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(16, 60, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(n.KernelError, match="multiple of 8"):
        n.skinny_linear(x, w, torch.empty(2, 16, dtype=torch.float32, device=DEV))
    with pytest.raises(n.KernelError, match="head_dim"):
        i32 = torch.zeros(1, dtype=torch.int32, device=DEV)
        q = torch.zeros(1, 24, dtype=torch.float32, device=DEV)
        n.attention_rows(q, 24, q, q, 24, None, None, None, 8, 0, i32, i32, i32, i32, i32,
                         torch.empty(1, 24, device=DEV), None, 1, 1, 24, 1.0, 0.0, 0, 1)


# ---------------------------------------------------------------- sampling

def _xorshift_uniforms(seed, count):
    rng = plain.XorShift64(seed)
    return [rng.next_f32() for _ in range(count)]


@pytest.mark.parametrize("vocab", [17, 300, 5000])
def test_greedy_takes_the_first_maximum(vocab):
    n = _native()
    g = torch.Generator().manual_seed(6)
    logits = torch.randn(6, vocab, generator=g)
    logits[2, 3] = logits[2, vocab - 2] = 50.0      # a tie: the lower index wins
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    n.sample_rows(logits.to(DEV), 0.0, 0, 1.0, None, out)
    assert out.tolist() == [plain.argmax(r.tolist()) for r in logits]
    assert out[2] == 3


@pytest.mark.parametrize("temperature,top_k,top_p", [
    (0.8, 0, 1.0), (1.3, 5, 1.0), (0.7, 0, 0.9), (1.0, 40, 0.95), (2.0, 1, 1.0), (0.5, 3, 0.3),
    (1.0, 400, 0.9), (1.5, 256, 1.0), (0.9, 257, 0.99), (0.3, 0, 0.9), (0.4, 0, 0.999), (3.0, 0, 0.5)])
def test_sampling_matches_the_plain_sampler_draw_by_draw(temperature, top_k, top_p):
    """Same generator, same draws: the kernel picks the token the plain sampler
    picks, except where a draw falls within rounding of a boundary."""
    n = _native()
    g = torch.Generator().manual_seed(7)
    vocab, rows, draws = 1000, 4, 40
    logits = torch.randn(rows, vocab, generator=g) * 3
    logits[1, 10] = logits[1, 20] = logits[1, 30] = logits[1].max() + 1   # ties at the top
    seeds = [42, 0, 7, 123456789]
    state = torch.tensor([s or 1 for s in seeds], dtype=torch.int64, device=DEV)
    dev_logits = logits.to(DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    got = []
    for _ in range(draws):
        n.sample_rows(dev_logits, temperature, top_k, top_p, state, out)
        got.append(out.tolist())
    differ = 0
    for r in range(rows):
        rng = plain.XorShift64(seeds[r])
        for d in range(draws):
            want = plain.sample_token(logits[r], temperature, top_k, top_p, rng)
            differ += want != got[d][r]
    assert differ <= 2, f"{differ} of {rows * draws} draws differ from the plain sampler"


@pytest.mark.parametrize("n_top,top_k,top_p", [(100, 7, 1.0), (100, 7, 0.5), (300, 7, 0.9), (1000, 5, 0.9),
                                                (3, 40, 0.95)])
def test_sampling_with_ties_at_the_edge_of_top_k(n_top, top_k, top_p):
    """Many equal logits at the k-th place: the lowest indices stay (few ties go through the
    sorted list, more than it holds through the general search)."""
    n = _native()
    g = torch.Generator().manual_seed(9)
    vocab, draws = 1000, 60
    logits = torch.randn(2, vocab, generator=g)
    where = torch.randperm(vocab, generator=g)[:n_top]
    logits[0, where] = 4.0
    logits[1, where] = 4.0
    logits[1, int(where[0])] = 6.0       # one above the ties
    seeds = [11, 12]
    state = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    dev = logits.to(DEV)
    out = torch.empty(2, dtype=torch.int32, device=DEV)
    got = []
    for _ in range(draws):
        n.sample_rows(dev, 0.9, top_k, top_p, state, out)
        got.append(out.tolist())
    differ = 0
    for r in range(2):
        rng = plain.XorShift64(seeds[r])
        for d in range(draws):
            differ += plain.sample_token(logits[r], 0.9, top_k, top_p, rng) != got[d][r]
    assert differ <= 2, f"{differ} of {2 * draws} draws differ from the plain sampler"


def test_sampling_at_the_vocabulary_of_the_real_model():
    n = _native()
    g = torch.Generator().manual_seed(10)
    vocab, rows, draws = 256000, 3, 12
    # (sharp enough that the sets the filters keep are hundreds of tokens, not a hundred thousand:
    # the plain sampler adds the probabilities one by one in 32-bit, which drifts over so many)
    logits = torch.randn(rows, vocab, generator=g) * 6.0
    seeds = [5, 6, 7]
    dev = logits.to(DEV)
    for temperature, top_k, top_p in ((0.8, 40, 0.95), (1.0, 0, 0.9), (0.7, 300, 1.0)):
        state = torch.tensor(seeds, dtype=torch.int64, device=DEV)
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        got = []
        for _ in range(draws):
            n.sample_rows(dev, temperature, top_k, top_p, state, out)
            got.append(out.tolist())
        differ = 0
        for r in range(rows):
            rng = plain.XorShift64(seeds[r])
            for d in range(draws):
                differ += plain.sample_token(logits[r], temperature, top_k, top_p, rng) != got[d][r]
        assert differ <= 2, f"{differ} of {rows * draws} draws differ ({temperature}, {top_k}, {top_p})"


def test_sampling_uses_the_indexed_generator_and_advances_it():
    n = _native()
    logits = torch.randn(2, 50, generator=torch.Generator().manual_seed(8)).to(DEV)
    state = torch.tensor([5, 6, 7, 8], dtype=torch.int64, device=DEV)
    out = torch.empty(2, dtype=torch.int32, device=DEV)
    n.sample_rows(logits, 1.0, 0, 1.0, state, out, torch.tensor([3, 1], dtype=torch.int32, device=DEV))
    after = state.tolist()
    r8, r6 = plain.XorShift64(8), plain.XorShift64(6)
    r8.next_u64(), r6.next_u64()
    assert after[0] == 5 and after[2] == 7
    assert after[3] & 0xFFFFFFFFFFFFFFFF == r8.state and after[1] & 0xFFFFFFFFFFFFFFFF == r6.state
