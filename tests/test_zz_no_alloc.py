"""sib_attention_decode_no_alloc, called the way its users call it: through the
exported C symbol, with raw device pointers, without any help from this
package's Python wrappers.

The entry point is for hosts that cannot allocate device memory when they call
(a C program without an allocator, a process whose memory is all in pools, a
loop in which cudaMalloc's wait for the device is not acceptable): the partial
results of the key splits live in an 8 MiB array inside the library instead of
in memory the caller passes.  The checks: on calls in a row, with different
inputs, shapes and numbers of splits, it gives what the ordinary entry point
gives with caller-provided scratch memory and what the plain implementation of
the tests computes (the array keeps the earlier calls' contents, which must not
leak into a later one: a small call is followed by one whose ticket counters
reach further than the small call's whole use of the array); a request larger
than the array is refused before anything is launched.

This file is collected last on purpose: a run that stops at the first failure
has then already run every other test.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

import plain_gemma2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _library():
    from strata_inference_b200.csrc.build import ensure_built
    lib = ctypes.CDLL(ensure_built())
    lib.sib_last_error.restype = ctypes.c_char_p
    lib.sib_attention_decode_no_alloc_floats.restype = c_longlong
    return lib


def _case(seed, rows, nh, nkv, hd, lengths, page=16):
    """Random queries, a paged cache holding `lengths[i]` positions for row i's
    sequence (slot i), and the index tensors of a single-token step."""
    g = torch.Generator().manual_seed(seed)
    pages_per_seq = -(-max(lengths) // page)
    n_pages = rows * pages_per_seq
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    table = perm.view(rows, pages_per_seq).contiguous()
    k_pool = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16)
    v_pool = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(rows, nh * hd, generator=g).to(torch.bfloat16)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    return dict(q=q.to(DEV), k=k_pool.to(DEV), v=v_pool.to(DEV), table=table.to(DEV),
                row_pos=i32([n - 1 for n in lengths]), row_seq=i32(list(range(rows))),
                seq_slot=i32(list(range(rows))), page=page, pages_per_seq=pages_per_seq)


def _call(lib, symbol, c, rows, nh, nkv, hd, scale, cap, window, splits, scratch=None):
    out = torch.full((rows, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    p = lambda t: c_void_p(t.data_ptr())  # noqa: E731
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    head = [p(c["q"]), c_int(nh * hd), p(c["k"]), p(c["v"]), p(c["table"]),
            c_int(c["pages_per_seq"]), c_int(c["page"]), c_int(0), p(c["row_pos"]),
            p(c["row_seq"]), p(c["seq_slot"]), p(out)]
    if scratch is not None:      # the ordinary entry point: its caller brings both
        tickets = torch.zeros(rows * nkv, dtype=torch.int32, device=DEV)
        head += [p(scratch), p(tickets)]
    tail = [c_int(rows), c_int(nh), c_int(nkv), c_int(hd), c_float(scale), c_float(cap),
            c_int(window), c_int(splits)]
    if scratch is not None:
        tail.append(c_int(4))    # warps a block; the entry point under test always takes 4
    tail.append(stream)
    rc = getattr(lib, symbol)(*head, *tail)
    torch.cuda.synchronize()
    return rc, out


def _plain_rows(c, lengths, nh, nkv, hd, scale, cap, window):
    """What tests/plain_gemma2.py's attention gives for each row: the sequence's keys and
    values are gathered from the pages, the query is the last position of a whole
    sequence whose other queries do not matter."""
    page = c["page"]
    out = []
    for i, n in enumerate(lengths):
        pages = c["table"][i].cpu().tolist()
        k = torch.cat([c["k"][p].cpu() for p in pages], dim=1)[:, :n].transpose(0, 1).double()
        v = torch.cat([c["v"][p].cpu() for p in pages], dim=1)[:, :n].transpose(0, 1).double()
        q = torch.zeros(n, nh, hd, dtype=torch.float64)
        q[n - 1] = c["q"][i].cpu().double().view(nh, hd)
        out.append(plain.attention(q, k.contiguous(), v.contiguous(), scale, cap, window)[n - 1]
                   .reshape(nh * hd))
    return torch.stack(out)


def test_no_alloc_entry_point_matches_the_ordinary_one_on_calls_in_a_row():
    lib = _library()
    nh, nkv, hd = 8, 4, 256
    scale = 2.0 / math.sqrt(hd)
    g = torch.Generator().manual_seed(9)
    many = torch.randint(20, 200, (32,), generator=g).tolist()
    calls = [  # (seed, sequence lengths, window, soft cap, splits)
        (1, [300, 17, 1024, 64], 0, 50.0, 7),
        (2, [90, 500], 128, 0.0, 3),
        # 32 rows x 4 kv heads: ticket counters 0..127, beyond the 64 words that the
        # calls above touched in front of their partial results
        (3, many, 0, 30.0, 3),
        (4, [700, 33, 64], 64, 50.0, 5),
    ]
    for seed, lengths, window, cap, splits in calls:
        rows = len(lengths)
        c = _case(seed, rows, nh, nkv, hd, lengths)
        need = lib.sib_attention_decode_no_alloc_floats(c_int(rows), c_int(nh), c_int(hd),
                                                        c_int(splits))
        # partial results behind a ticket region of a fixed size
        assert need == rows * nh * splits * (hd + 2) + 4096
        scratch = torch.empty(need, dtype=torch.float32, device=DEV)
        rc, want = _call(lib, "sib_attention_decode", c, rows, nh, nkv, hd, scale, cap, window,
                         splits, scratch)
        assert rc == 0, lib.sib_last_error().decode()
        rc, got = _call(lib, "sib_attention_decode_no_alloc", c, rows, nh, nkv, hd, scale, cap,
                        window, splits)
        assert rc == 0, lib.sib_last_error().decode()
        assert torch.isfinite(got.float()).all(), f"call with seed {seed}: rows were not written"
        scale_of = want.float().abs().max().item()
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 1e-2 * scale_of, f"call with seed {seed}: {err:.3e} vs {scale_of:.3e}"
        ref = _plain_rows(c, lengths, nh, nkv, hd, scale, cap, window)
        err = (got.double().cpu() - ref).abs().max().item()
        assert err <= 1e-2 * ref.abs().max().item(), f"call with seed {seed} vs plain: {err:.3e}"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _library()
    nh, nkv, hd = 8, 4, 256
    rows, splits = 64, 128                     # 64 * 8 * 128 * 258 floats: far beyond 8 MiB
    c = _case(3, rows, nh, nkv, hd, [32] * rows)
    rc, out = _call(lib, "sib_attention_decode_no_alloc", c, rows, nh, nkv, hd, 0.1, 0.0, 0, splits)
    assert rc != 0
    msg = lib.sib_last_error().decode()
    assert "built-in array holds" in msg and str(rows * nh * splits * (hd + 2) + 4096) in msg
    assert torch.isnan(out.float()).all()      # nothing was launched
    # more (row, kv head) pairs than ticket counters, although the partial results would fit
    rows, splits = 1100, 2
    c = _case(4, rows, 4, 4, 64, [16] * rows)
    rc, out = _call(lib, "sib_attention_decode_no_alloc", c, rows, 4, 4, 64, 0.1, 0.0, 0, splits)
    assert rc != 0 and "ticket counters" in lib.sib_last_error().decode()
    assert torch.isnan(out.float()).all()
