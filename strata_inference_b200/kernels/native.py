"""The compiled sm_100a kernels, called with torch tensors.

The library is plain C (``csrc/*.cu``), loaded with ctypes; each wrapper
checks types and layouts, passes raw device pointers and the current
stream, and raises :class:`KernelError` with the library's message when a
launcher refuses its arguments.  There is no other implementation behind
these functions: without the compiled library, or on a device that is not
sm_100, they raise.
"""

from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

F32, BF16 = 0, 1
EPI_NONE, EPI_SOFTCAP, EPI_GEGLU = 0, 1, 2
ROPE_HALF_SPLIT, ROPE_INTERLEAVED = 0, 1

_lib = None


class KernelError(RuntimeError):
    pass


def library():
    """Load (compiling first if needed) the kernel library."""
    global _lib
    if _lib is not None:
        return _lib
    from ..csrc.build import ensure_built
    path = ensure_built()
    lib = ctypes.CDLL(path)
    lib.sib_last_error.restype = ctypes.c_char_p
    lib.sib_attention_rows_scratch_bytes.restype = c_longlong
    if lib.sib_compiled_arch() != 100:
        raise KernelError(f"{path} was not compiled for sm_100a")
    _lib = lib
    return lib


def require_device(device: torch.device) -> None:
    """Fail loudly unless ``device`` is a CUDA device of compute capability 10.x."""
    if device.type != "cuda" or not torch.cuda.is_available():
        raise KernelError("strata_inference_b200 runs on an sm_100 CUDA device only; "
                          f"got device '{device}' (there is no CPU path)")
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise KernelError(f"strata_inference_b200 is compiled for sm_100a; device '{device}' "
                          f"has compute capability {major}.{minor}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream of the current device (asked for at every launch: it changes
    under graph capture).  torch's raw getter costs a fraction of a microsecond, the Stream
    object several."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {dtype} is not supported (float32 and bfloat16 are)")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_launches = 0


def launch_count() -> int:
    """How many launcher calls of this library succeeded so far in this process
    (a launcher that merges split partial results launches two kernels and counts once)."""
    return _launches


def _check(rc: int) -> None:
    global _launches
    if rc != 0:
        raise KernelError(library().sib_last_error().decode())
    _launches += 1


def _want(t: torch.Tensor, dtype: torch.dtype, name: str, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor")
    if t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: expected a contiguous tensor")


# --------------------------------------------------------------------------
# Per-kernel timing.  Inside ``with KernelProfile() as prof:`` every launcher of this
# module (and whatever else is wrapped in ``prof.region``) is bracketed by CUDA events;
# ``prof.rows()`` then gives, per kernel class, the calls, the device time and the bytes
# and operations that the work needs by its shapes.  Outside such a block the wrappers
# cost one comparison.  The reference's counterpart is a device synchronisation and a
# wall-clock figure per layer (src/model/layer.rs:1265,1365-1375).

_profile: Optional["KernelProfile"] = None
# Set while a chain of deferred steps is being collected (parts/base.py ProductChain): called
# before any other launch of this module, so that the chain's kernel runs first.
_pending: Optional[Callable[[], None]] = None


def set_pending(flush: Optional[Callable[[], None]]) -> None:
    global _pending
    _pending = flush


class KernelProfile:
    """``plan``: an earlier profile of the same launch sequence.  With a plan the events
    are made for recording inside a CUDA graph (they are re-recorded by every replay) and
    each launch takes its kernel class and work from the plan, in order, instead of
    working them out (which may read device memory and cannot be done while capturing)."""

    def __init__(self, plan: Optional["KernelProfile"] = None):
        self.events: List[Tuple[str, torch.cuda.Event, torch.cuda.Event, float, float]] = []
        self.plan = [(n, b, f) for n, _, _, b, f in plan.events] if plan is not None else None
        self._next = 0

    def __enter__(self) -> "KernelProfile":
        global _profile
        self._outer, _profile = _profile, self
        return self

    def __exit__(self, *exc) -> None:
        global _profile
        _profile = self._outer

    def planned(self) -> Tuple[str, float, float]:
        item = self.plan[self._next % len(self.plan)]
        self._next += 1
        return item

    def region(self, name: str, nbytes: float, flops: float):
        return _Region(self, name, nbytes, flops)

    def rows(self, last: Optional[int] = None) -> List[Dict]:
        """One row per kernel class, longest first (synchronises the device).  ``last``:
        only the last so many launches (the ones a graph replays)."""
        torch.cuda.synchronize()
        table: Dict[str, Dict] = {}
        for name, start, end, nbytes, flops in (self.events[-last:] if last else self.events):
            r = table.setdefault(name, {"name": name, "calls": 0, "ms": 0.0, "bytes": 0.0,
                                        "flops": 0.0})
            r["calls"] += 1
            r["ms"] += start.elapsed_time(end)
            r["bytes"] += nbytes
            r["flops"] += flops
        return sorted(table.values(), key=lambda r: -r["ms"])


class _Region:
    def __init__(self, prof, name, nbytes, flops):
        self.prof = prof
        if prof.plan is not None:
            name, nbytes, flops = prof.planned()
        self.name, self.nbytes, self.flops = name, nbytes, flops

    def __enter__(self):
        external = self.prof.plan is not None
        self.start = torch.cuda.Event(enable_timing=True, external=external)
        self.end = torch.cuda.Event(enable_timing=True, external=external)
        self.start.record()
        return self

    def __exit__(self, *exc):
        self.end.record()
        self.prof.events.append((self.name, self.start, self.end, float(self.nbytes),
                                 float(self.flops)))


def profile_region(name: str, nbytes: float, flops: float):
    """A region of the active profile, or nothing when none is active."""
    return _profile.region(name, nbytes, flops) if _profile is not None else _NO_REGION


class _NoRegion:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_REGION = _NoRegion()


def recording_allowed() -> bool:
    """False while a profile without a plan is active: its events and the work it reads
    from the device cannot go into a CUDA graph, so steps are not recorded meanwhile."""
    return _profile is None or _profile.plan is not None


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def _timed(work: Callable):
    """Wrap a launcher: under an active profile it is timed and ``work(*args)`` gives
    (kernel class, bytes, operations) from the call's arguments."""
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kw):
            if _pending is not None:
                _pending()          # deferred work that this launch may depend on goes first
            if _profile is None:
                return fn(*args, **kw)
            name, nbytes, flops = ("", 0, 0) if _profile.plan is not None else work(*args, **kw)
            with _profile.region(name, nbytes, flops):
                return fn(*args, **kw)
        return wrapper
    return deco


def _attention_cache_work(kind, row_pos, k_pool, n_heads, head_dim, window, rows, value_dim=None):
    """Keys and values a row at ``row_pos`` reads from the cache (reads the positions back:
    only done under a profile)."""
    seen = row_pos.to(torch.int64) + 1
    if window > 0:
        seen = seen.clamp(max=window)
    keys = int(seen.sum().item())
    n_kv = k_pool.shape[1]
    nbytes = keys * n_kv * (head_dim + (value_dim or head_dim)) * k_pool.element_size()
    return kind, nbytes, 4.0 * keys * n_heads * head_dim


def _prompt_work(kind, qkv, seq_len, n_heads, head_dim, window):
    """Prompts from position 0: (query, key) pairs inside the causal mask and the window."""
    pairs = 0
    for n in seq_len.to(torch.int64).tolist():
        if window and n > window:
            pairs += window * (window + 1) // 2 + (n - window) * window
        else:
            pairs += n * (n + 1) // 2
    return kind, _nbytes(qkv) + qkv.shape[0] * n_heads * head_dim * qkv.element_size(), \
        4.0 * pairs * n_heads * head_dim


# --------------------------------------------------------------------------

@_timed(lambda tokens, table, scale, out: ("embed_rows", 2 * _nbytes(out), 0))
def embed_rows(tokens: torch.Tensor, table: torch.Tensor, scale: float,
               out: torch.Tensor) -> torch.Tensor:
    """out[r] = scale * table[tokens[r]] in 32-bit."""
    _want(tokens, torch.int32, "tokens")
    _want(out, torch.float32, "out")
    rows, hidden = out.shape
    if tokens.numel() != rows or table.shape[1] != hidden or not table.is_contiguous():
        raise KernelError("embed_rows: shapes do not fit")
    _check(library().sib_embed_rows(_ptr(tokens), _ptr(table), _code(table.dtype), _ptr(out),
                                    c_int(rows), c_int(hidden), c_float(scale), _stream()))
    return out


def randn_fill(dst: torch.Tensor, rows: int, cols: int, group: int, group_stride: int, key: int,
               offset: float, std: float, stored_dtype: torch.dtype) -> None:
    """Seeded normal values for a stored tensor of [rows, cols], written to ``dst``: a view
    [runs, rows a run, cols] into the weight buffer whose runs may lie apart (see
    csrc/randn_fill.cu).  ``key`` is the tensor's 64-bit key."""
    if not dst.is_cuda or dst.stride(2) != 1 or dst.stride(1) != cols:
        raise KernelError("randn_fill: destination runs must be rows of `cols` contiguous elements")
    runs, per_run, _ = dst.shape
    if runs * per_run != rows or (runs > 1 and (per_run != group or dst.stride(0) != group_stride * cols)):
        raise KernelError("randn_fill: the destination view does not fit the run layout")
    _check(library().sib_randn_fill(
        _ptr(dst), _code(dst.dtype), c_longlong(rows), c_longlong(cols),
        c_longlong(group if runs > 1 else 0), c_longlong(group_stride if runs > 1 else 0),
        ctypes.c_ulonglong(key), c_float(offset), c_float(std),
        c_int(BF16 if stored_dtype == torch.bfloat16 else F32), _stream()))


@_timed(lambda gate_up, out, group=0: ("gelu_mul", _nbytes(gate_up, out), 0))
def gelu_mul(gate_up: torch.Tensor, out: torch.Tensor, group: int = 0) -> torch.Tensor:
    """out[r, i] = gelu_tanh(gate(r, i)) * up(r, i); gate_up rows are [gates | ups]
    (group 0) or groups of ``group`` gates followed by their ups."""
    rows, inter = out.shape
    _want(gate_up, out.dtype, "gate_up")
    _want(out, out.dtype, "out")
    if tuple(gate_up.shape) != (rows, 2 * inter):
        raise KernelError("gelu_mul: gate_up must be [rows, 2 * intermediate]")
    _check(library().sib_gelu_mul(_ptr(gate_up), _ptr(out), _code(out.dtype), c_int(rows),
                                  c_int(inter), c_int(group), _stream()))
    return out


@_timed(lambda x, cap: ("softcap", 2 * _nbytes(x), 0))
def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap) in place (32-bit)."""
    _want(x, torch.float32, "x")
    _check(library().sib_softcap(_ptr(x), c_longlong(x.numel()), c_float(cap), _stream()))
    return x


@_timed(lambda x, gain, eps, out, rows=None: (
    "rms_norm", out.shape[0] * x.shape[1] * x.element_size() + _nbytes(out), 0))
def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = rms(x[rows[i] if rows else i]) * gain; statistics in 32-bit."""
    _want(gain, torch.float32, "gain")
    _want(x, x.dtype, "x")
    _want(out, out.dtype, "out")
    n, hidden = out.shape
    if x.shape[1] != hidden or gain.numel() != hidden:
        raise KernelError("rms_norm: shapes do not fit")
    if rows is not None:
        _want(rows, torch.int32, "rows")
        if rows.numel() != n:
            raise KernelError("rms_norm: one row index per output row")
    elif x.shape[0] != n:
        raise KernelError("rms_norm: x and out differ in rows")
    _check(library().sib_rms_norm(_ptr(x), _code(x.dtype), _ptr(rows), _ptr(gain), c_float(eps),
                                  _ptr(out), _code(out.dtype), c_int(n), c_int(hidden), _stream()))
    return out


@_timed(lambda a, post_gain, post_eps, h, pre_gain, pre_eps, out: (
    "add_rms_norm", _nbytes(a, out) + 2 * _nbytes(h), 0))
def add_rms_norm(a: torch.Tensor, post_gain: Optional[torch.Tensor], post_eps: float,
                 h: torch.Tensor, pre_gain: Optional[torch.Tensor], pre_eps: float,
                 out: Optional[torch.Tensor]) -> None:
    """h += rms(a) * post_gain (or a when post_gain is None); out = rms(h) * pre_gain."""
    _want(h, torch.float32, "h")
    _want(a, a.dtype, "a")
    rows, hidden = h.shape
    if tuple(a.shape) != (rows, hidden):
        raise KernelError("add_rms_norm: a and h differ in shape")
    for g, nm in ((post_gain, "post_gain"), (pre_gain, "pre_gain")):
        if g is not None:
            _want(g, torch.float32, nm)
            if g.numel() != hidden:
                raise KernelError(f"add_rms_norm: {nm} has the wrong length")
    if pre_gain is not None:
        if out is None:
            raise KernelError("add_rms_norm: pre_gain needs out")
        _want(out, a.dtype, "out")
    _check(library().sib_add_rms_norm(_ptr(a), _code(a.dtype), _ptr(post_gain), c_float(post_eps),
                                      _ptr(h), _ptr(pre_gain), c_float(pre_eps), _ptr(out),
                                      c_int(rows), c_int(hidden), _stream()))


@_timed(lambda qkv, *a, **kw: ("rope_store", 2 * _nbytes(qkv), 0))
def rope_store(qkv: torch.Tensor, row_pos, row_seq, seq_slot, seq_end,
               inv_freq: Optional[torch.Tensor], rotary_dim: int, style: int,
               k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
               page_table: Optional[torch.Tensor], page_tokens: int, ring_tokens: int,
               n_heads: int, n_kv: int, head_dim: int) -> None:
    """Rotate q and k of the packed rows in place and write k, v into the paged cache."""
    _want(qkv, qkv.dtype, "qkv")
    rows = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("rope_store: qkv width does not fit the head counts")
    if inv_freq is not None:
        _want(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("rope_store: one frequency per rotated pair")
    max_pages = 0
    if k_pool is not None:
        _want(k_pool, qkv.dtype, "k_pool")
        _want(v_pool, qkv.dtype, "v_pool")
        _want(page_table, torch.int32, "page_table")
        max_pages = page_table.shape[1]
        if tuple(k_pool.shape[1:]) != (n_kv, page_tokens, head_dim):
            raise KernelError("rope_store: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
    _check(library().sib_rope_store(
        _ptr(qkv), _code(qkv.dtype), _ptr(row_pos), _ptr(row_seq), _ptr(seq_slot), _ptr(seq_end),
        _ptr(inv_freq), c_int(rotary_dim), c_int(style), _ptr(k_pool), _ptr(v_pool),
        _ptr(page_table), c_int(max_pages), c_int(page_tokens), c_int(ring_tokens), c_int(rows),
        c_int(n_heads), c_int(n_kv), c_int(head_dim), _stream()))


def attention_rows_scratch_bytes(rows: int, n_heads: int, head_dim: int, splits: int) -> int:
    return int(library().sib_attention_rows_scratch_bytes(c_int(rows), c_int(n_heads),
                                                          c_int(head_dim), c_int(splits)))


@_timed(lambda q, q_stride, k_new, v_new, kv_stride, k_pool, v_pool, page_table, page_tokens,
        ring_tokens, row_pos, row_seq, seq_slot, seq_start, seq_row0, out, scratch, n_heads, n_kv,
        head_dim, scale, softcap, window, splits: (
            _attention_cache_work("attention_rows (cache)", row_pos, k_pool, n_heads, head_dim,
                                  window, out.shape[0]) if k_pool is not None else
            ("attention_rows (prompt)", 2 * _nbytes(out) * (1 + 2 * n_kv / n_heads),
             2.0 * (row_pos.to(torch.int64) + 1).sum().item() * 2 * n_heads * head_dim)))
def attention_rows(q: torch.Tensor, q_stride: int, k_new: Optional[torch.Tensor],
                   v_new: Optional[torch.Tensor], kv_stride: int,
                   k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                   page_table: Optional[torch.Tensor], page_tokens: int, ring_tokens: int,
                   row_pos, row_seq, seq_slot, seq_start, seq_row0, out: torch.Tensor,
                   scratch: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int,
                   scale: float, softcap: float, window: int, splits: int) -> torch.Tensor:
    """General attention of independent rows (see csrc/attention_rows.cu).

    ``q``, ``k_new``, ``v_new`` may be views into one packed buffer; only
    their first elements' addresses and the strides are used."""
    rows = out.shape[0]
    _want(out, out.dtype, "out")
    if q.dtype != out.dtype:
        raise KernelError("attention_rows: q and out differ in type")
    max_pages = page_table.shape[1] if page_table is not None else 0
    if k_pool is not None and tuple(k_pool.shape[1:]) != (n_kv, page_tokens, head_dim):
        raise KernelError("attention_rows: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
    if splits > 1:
        need = attention_rows_scratch_bytes(rows, n_heads, head_dim, splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelError(f"attention_rows: {need} bytes of scratch memory are needed")
    _check(library().sib_attention_rows(
        _ptr(q), c_int(q_stride), _ptr(k_new), _ptr(v_new), c_int(kv_stride), _ptr(k_pool),
        _ptr(v_pool), _ptr(page_table), c_int(max_pages), c_int(page_tokens), c_int(ring_tokens),
        _ptr(row_pos), _ptr(row_seq), _ptr(seq_slot), _ptr(seq_start), _ptr(seq_row0), _ptr(out),
        _ptr(scratch), _code(out.dtype), c_int(rows), c_int(n_heads), c_int(n_kv), c_int(head_dim),
        c_float(scale), c_float(softcap), c_int(window), c_int(splits), _stream()))
    return out


def attention_decode_supports(n_heads: int, n_kv: int, head_dim: int, page_tokens: int) -> bool:
    return bool(library().sib_attention_decode_supports(c_int(n_heads), c_int(n_kv),
                                                        c_int(head_dim), c_int(page_tokens)))


def attention_decode_resident_warps(n_heads: int, n_kv: int, head_dim: int, warps: int = 4) -> int:
    """Warps of the decode attention kernel that the current device holds at a time for this
    shape, in blocks of ``warps`` warps (0: not a shape the kernel takes)."""
    return int(library().sib_attention_decode_resident_warps_of(c_int(n_heads), c_int(n_kv),
                                                                c_int(head_dim), c_int(warps)))


@_timed(lambda q, q_stride, k_pool, v_pool, page_table, page_tokens, ring_tokens, row_pos, row_seq,
        seq_slot, out, scratch, tickets, n_heads, n_kv, head_dim, scale, softcap, window, splits,
        warps=4, fresh=0: _attention_cache_work("attention_decode", row_pos, k_pool, n_heads,
                                                head_dim, window, out.shape[0]))
def attention_decode(q: torch.Tensor, q_stride: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                     page_table: torch.Tensor, page_tokens: int, ring_tokens: int, row_pos,
                     row_seq, seq_slot, out: torch.Tensor, scratch: Optional[torch.Tensor],
                     tickets: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int,
                     scale: float, softcap: float, window: int, splits: int,
                     warps: int = 4, fresh: int = 0) -> torch.Tensor:
    """Attention of single rows over the bfloat16 cache (see csrc/attention_decode.cu).
    ``splits`` blocks of ``warps`` warps share the keys of a (row, kv head); with more than one they
    need ``scratch`` for their partial results and ``tickets``: int32 counters, one
    per (row, kv head), zero before the first call (every call leaves them zero).
    ``fresh``: the most positions of a sequence that the kernel before this one wrote (the
    rows a sequence has in this step); keys below them are fetched while that kernel still
    runs.  0: every load waits for it."""
    global _launches
    rows = out.shape[0]
    _want(out, torch.bfloat16, "out")
    _want(k_pool, torch.bfloat16, "k_pool")
    _want(v_pool, torch.bfloat16, "v_pool")
    _want(page_table, torch.int32, "page_table")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode: q must be bfloat16")
    if tuple(k_pool.shape[1:]) != (n_kv, page_tokens, head_dim):
        raise KernelError("attention_decode: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
    if splits > 1:
        need = attention_rows_scratch_bytes(rows, n_heads, head_dim, splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelError(f"attention_decode: {need} bytes of scratch memory are needed")
        if tickets is None or tickets.dtype != torch.int32 or tickets.numel() < rows * n_kv:
            raise KernelError(f"attention_decode: {rows * n_kv} int32 ticket counters are needed")
    _check(library().sib_attention_decode_fresh(
        _ptr(q), c_int(q_stride), _ptr(k_pool), _ptr(v_pool), _ptr(page_table),
        c_int(page_table.shape[1]), c_int(page_tokens), c_int(ring_tokens), _ptr(row_pos),
        _ptr(row_seq), _ptr(seq_slot), _ptr(out), _ptr(scratch), _ptr(tickets), c_int(rows),
        c_int(n_heads), c_int(n_kv), c_int(head_dim), c_float(scale), c_float(softcap),
        c_int(window), c_int(splits), c_int(warps), c_int(fresh), _stream()))
    return out


def attention_prefill_supports(n_heads: int, n_kv: int, head_dim: int) -> bool:
    return bool(library().sib_attention_prefill_supports(c_int(n_heads), c_int(n_kv),
                                                         c_int(head_dim)))


@_timed(lambda qkv, out, seq_row0, seq_len, n_seqs, max_len, n_heads, n_kv, head_dim, scale,
        softcap, window: _prompt_work("attention_prefill (mma.sync)", qkv, seq_len, n_heads,
                                      head_dim, window))
def attention_prefill(qkv: torch.Tensor, out: torch.Tensor, seq_row0, seq_len, n_seqs: int,
                      max_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                      softcap: float, window: int) -> torch.Tensor:
    """Attention of packed bfloat16 prompts that start at position 0 over their
    own (rotated) keys and values (see csrc/attention_prefill.cu)."""
    _want(qkv, torch.bfloat16, "qkv")
    _want(out, torch.bfloat16, "out")
    if out.shape[0] != qkv.shape[0] or out.shape[1] != n_heads * head_dim:
        raise KernelError("attention_prefill: out must be [rows, heads * head_dim]")
    _check(library().sib_attention_prefill(
        _ptr(qkv), c_int(qkv.shape[1]), _ptr(out), _ptr(seq_row0), _ptr(seq_len), c_int(n_seqs),
        c_int(max_len), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_float(scale),
        c_float(softcap), c_int(window), _stream()))
    return out


def attention_prefill_tc_supports(n_heads: int, n_kv: int, head_dim: int, width: int) -> bool:
    return bool(library().sib_attention_prefill_tc_supports(c_int(n_heads), c_int(n_kv),
                                                            c_int(head_dim), c_int(width)))


def attention_prefill_tc_split(n_seqs: int, max_len: int, n_heads: int, n_kv: int,
                               head_dim: int):
    """(bytes of scratch memory, ticket counters) that a launch of this shape needs to split
    its long blocks of query rows; (0, 0) if it would not split."""
    nbytes, n_tickets = c_longlong(0), c_int(0)
    from ctypes import byref
    library().sib_attention_prefill_tc_split(c_int(n_seqs), c_int(max_len), c_int(n_heads),
                                             c_int(n_kv), c_int(head_dim), byref(nbytes),
                                             byref(n_tickets))
    return int(nbytes.value), int(n_tickets.value)


def attention_prefill_tc_plan(lens: Sequence[int], n_heads: int, n_kv: int, head_dim: int,
                              window: int, first_query: Optional[Sequence[int]] = None):
    """(work items, bytes of scratch memory, ticket counters) of a launch for prompts of these
    lengths that runs as a balanced list of work items; (0, 0, 0) if it would run as a grid.
    ``first_query``: per sequence, the position from which rows are queries."""
    from ctypes import byref
    nbytes, n_tickets = c_longlong(0), c_int(0)
    arr = (c_int * len(lens))(*[int(n) for n in lens])
    q0 = None if first_query is None else (c_int * len(lens))(*[int(n) for n in first_query])
    n_items = library().sib_attention_prefill_tc_plan(arr, q0, c_int(len(lens)), c_int(n_heads),
                                                      c_int(n_kv), c_int(head_dim), c_int(window),
                                                      byref(nbytes), byref(n_tickets))
    return int(n_items), int(nbytes.value), int(n_tickets.value)


@_timed(lambda qkv, out, seq_row0, seq_len, n_seqs, max_len, n_heads, n_kv, head_dim, scale,
        softcap, window, scratch=None, tickets=None, host_lens=None, seq_q0=None,
        host_q0=None: _prompt_work(
            "attention_prefill_tc (tcgen05)", qkv, seq_len, n_heads, head_dim, window))
def attention_prefill_tc(qkv: torch.Tensor, out: torch.Tensor, seq_row0, seq_len, n_seqs: int,
                         max_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                         softcap: float, window: int, scratch: Optional[torch.Tensor] = None,
                         tickets: Optional[torch.Tensor] = None,
                         host_lens: Optional[Sequence[int]] = None,
                         seq_q0: Optional[torch.Tensor] = None,
                         host_q0: Optional[Sequence[int]] = None) -> torch.Tensor:
    """The prompt attention on tcgen05 (see csrc/attention_prefill_tc.cu).  With ``scratch``
    and ``tickets`` (int32, zero before the first call; every call leaves them zero) of the
    sizes ``attention_prefill_tc_split`` gives, a launch that cannot fill the device runs its
    long blocks of query rows as two halves.  With ``host_lens`` (the prompts' lengths, as
    ``seq_len`` holds them on the device) and memory of the sizes ``attention_prefill_tc_plan``
    gives, the launch is a list of work items ordered by their work, with the blocks split
    that make the busiest SM's share smallest.  ``seq_q0`` (int32 on the device, ``host_q0``
    the same on the host): per sequence the position from which rows are queries; the rows
    before it bring keys and values only and their output rows are not written."""
    _want(qkv, torch.bfloat16, "qkv")
    _want(out, torch.bfloat16, "out")
    if out.shape[0] != qkv.shape[0] or out.shape[1] != n_heads * head_dim:
        raise KernelError("attention_prefill_tc: out must be [rows, heads * head_dim]")
    if tickets is not None:
        _want(tickets, torch.int32, "tickets")
    _check(library().sib_attention_prefill_tc(
        _ptr(qkv), c_int(qkv.shape[1]), c_int(qkv.shape[0]), _ptr(out), _ptr(seq_row0),
        _ptr(seq_len), c_int(n_seqs), c_int(max_len), c_int(n_heads), c_int(n_kv), c_int(head_dim),
        c_float(scale), c_float(softcap), c_int(window), _ptr(scratch),
        c_longlong(scratch.numel() * scratch.element_size() if scratch is not None else 0),
        _ptr(tickets), c_int(tickets.numel() if tickets is not None else 0),
        None if host_lens is None else (c_int * len(host_lens))(*[int(n) for n in host_lens]),
        _ptr(seq_q0),
        None if host_q0 is None else (c_int * len(host_q0))(*[int(n) for n in host_q0]),
        _stream()))
    return out


@_timed(lambda packed, k_pool, *a, **kw: ("gather_kv_rows", 0, 0))
def gather_kv_rows(packed: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   page_table: torch.Tensor, seq_slot: torch.Tensor, seq_from: torch.Tensor,
                   seq_upto: torch.Tensor, seq_row0: torch.Tensor, most: int, page_tokens: int,
                   ring_tokens: int, n_heads: int, n_kv: int, head_dim: int) -> torch.Tensor:
    """Keys and values of the positions [seq_from[b], seq_upto[b]) that sequence b holds in
    the paged cache, into rows seq_row0[b] + position of the packed q|k|v buffer (q columns
    of those rows: zero).  ``most``: the most positions of any sequence."""
    _want(packed, torch.bfloat16, "packed")
    _want(k_pool, torch.bfloat16, "k_pool")
    _want(v_pool, torch.bfloat16, "v_pool")
    for t, name in ((page_table, "page_table"), (seq_slot, "seq_slot"), (seq_from, "seq_from"),
                    (seq_upto, "seq_upto"), (seq_row0, "seq_row0")):
        _want(t, torch.int32, name)
    if packed.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("gather_kv_rows: the packed rows do not fit the head counts")
    _check(library().sib_gather_kv_rows(
        _ptr(packed), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(seq_slot), _ptr(seq_from),
        _ptr(seq_upto), _ptr(seq_row0), c_int(seq_slot.numel()), c_int(most), c_int(n_heads),
        c_int(n_kv), c_int(head_dim), c_int(page_table.shape[1]), c_int(page_tokens),
        c_int(ring_tokens), _stream()))
    return packed


def attention_prefill_tc_error(clear: bool = True) -> int:
    """0, or the code left by a block of attention_prefill_tc whose bounded wait ran out
    (synchronises the device)."""
    torch.cuda.synchronize()
    return int(library().sib_attention_prefill_tc_error(c_int(1 if clear else 0)))


SKINNY_MAX_ROWS = 64


def _product_work(kind, x, w, out):
    return (f"{kind} {w.shape[0]}x{w.shape[1]}", _nbytes(w, out) + x.shape[0] * x.shape[1]
            * x.element_size(), 2.0 * x.shape[0] * w.shape[0] * w.shape[1])


@_timed(lambda x, w, out, epilogue=EPI_NONE, cap=0.0: _product_work("skinny_linear", x, w, out))
def skinny_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                  cap: float = 0.0) -> torch.Tensor:
    """out = x . w^T for at most 64 rows of bfloat16 x (see csrc/linear_skinny.cu)."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, out.dtype, "out", contiguous=False)
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue == EPI_GEGLU else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("skinny_linear: shapes do not fit")
    _check(library().sib_skinny_linear(_ptr(w), _ptr(x), _ptr(out), _code(out.dtype), c_int(R),
                                       c_int(N), c_int(K), c_int(x.stride(0)),
                                       c_int(out.stride(0)), c_int(epilogue), c_float(cap),
                                       _stream()))
    return out


def linear_stream_supports(R: int, N: int, K: int, x_stride: int) -> bool:
    return bool(library().sib_linear_stream_supports(c_int(R), c_int(N), c_int(K), c_int(x_stride)))


@_timed(lambda x, w, out, epilogue=EPI_NONE, cap=0.0, ksplit=0, stages=0: _product_work(
    "linear_stream", x, w, out))
def linear_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                  cap: float = 0.0, ksplit: int = 0, stages: int = 0) -> torch.Tensor:
    """out = x . w^T for at most 16 rows of bfloat16 x, the weights staged through shared
    memory by TMA (see csrc/linear_stream.cu).  ``ksplit`` blocks of a cluster share a tile
    of weight rows, ``stages`` tiles are in flight per block; 0 lets the launcher choose."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, out.dtype, "out", contiguous=False)
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue == EPI_GEGLU else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear_stream: shapes do not fit")
    _check(library().sib_linear_stream(_ptr(w), _ptr(x), _ptr(out), _code(out.dtype), c_int(R),
                                       c_int(N), c_int(K), c_int(x.stride(0)),
                                       c_int(out.stride(0)), c_int(epilogue), c_float(cap),
                                       c_int(ksplit), c_int(stages), _stream()))
    return out


def linear_rows_tc_max_rows() -> int:
    return int(library().sib_linear_rows_tc_max_rows())


@_timed(lambda x, w, out, epilogue=EPI_NONE, cap=0.0, ksplit=0, stages=0: _product_work(
    "linear_rows_tc", x, w, out))
def linear_rows_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                   cap: float = 0.0, ksplit: int = 0, stages: int = 0) -> torch.Tensor:
    """out = x . w^T for at most 128 rows of bfloat16 x on the tcgen05 tensor cores, the
    weights streamed through a ring of TMA stages (see csrc/linear_rows_tc.cu).  ``ksplit``
    blocks of a cluster share a tile of 128 weight rows, ``stages`` stages are in flight per
    block; 0 lets the launcher choose."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, out.dtype, "out", contiguous=False)
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue == EPI_GEGLU else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear_rows_tc: shapes do not fit")
    _check(library().sib_linear_rows_tc(_ptr(w), _ptr(x), _ptr(out), _code(out.dtype), c_int(R),
                                        c_int(N), c_int(K), c_int(x.stride(0)),
                                        c_int(out.stride(0)), c_int(epilogue), c_float(cap),
                                        c_int(ksplit), c_int(stages), _stream()))
    return out


@_timed(lambda x, w, out, *a, **kw: _product_work("skinny_linear_rope", x, w, out))
def skinny_linear_rope(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_pos, row_seq,
                       seq_slot, seq_end, inv_freq: torch.Tensor,
                       k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                       page_table: Optional[torch.Tensor], page_tokens: int, ring_tokens: int,
                       n_heads: int, n_kv: int, head_dim: int) -> torch.Tensor:
    """The q|k|v product of at most 16 bfloat16 rows that also rotates q and k (half-split
    pairs over the whole head) and writes k and v into the paged cache as well as into
    ``out`` (see csrc/linear_skinny.cu, RopeTail).  ``n_kv == 0``: q rows only, nothing stored."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, torch.bfloat16, "out", contiguous=False)
    _want(inv_freq, torch.float32, "inv_freq")
    R, K = x.shape
    N = (n_heads + 2 * n_kv) * head_dim
    if tuple(w.shape) != (N, K) or tuple(out.shape) != (R, N) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("skinny_linear_rope: shapes do not fit the head counts")
    if inv_freq.numel() * 2 != head_dim:
        raise KernelError("skinny_linear_rope: one frequency per pair of the whole head")
    max_pages = 0
    if n_kv:
        _want(k_pool, torch.bfloat16, "k_pool")
        _want(v_pool, torch.bfloat16, "v_pool")
        _want(page_table, torch.int32, "page_table")
        max_pages = page_table.shape[1]
        if tuple(k_pool.shape[1:]) != (n_kv, page_tokens, head_dim):
            raise KernelError("skinny_linear_rope: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
    _check(library().sib_skinny_linear_rope(
        _ptr(w), _ptr(x), _ptr(out), c_int(R), c_int(K), c_int(x.stride(0)), c_int(out.stride(0)),
        _ptr(row_pos), _ptr(row_seq), _ptr(seq_slot), _ptr(seq_end), _ptr(inv_freq),
        _ptr(k_pool) if n_kv else c_void_p(0), _ptr(v_pool) if n_kv else c_void_p(0),
        _ptr(page_table) if n_kv else c_void_p(0), c_int(max_pages), c_int(page_tokens),
        c_int(ring_tokens), c_int(n_heads), c_int(n_kv), c_int(head_dim), _stream()))
    return out


def gemm_tcgen05_supports(R: int, N: int, K: int, x_stride: int) -> bool:
    return bool(library().sib_gemm_tcgen05_supports(c_int(R), c_int(N), c_int(K),
                                                    c_longlong(x_stride)))


@_timed(lambda x, w, out, epilogue=EPI_NONE, cap=0.0, one_block=False: _product_work(
    "gemm_tcgen05", x, w, out))
def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                 cap: float = 0.0, one_block: bool = False) -> torch.Tensor:
    """out = x . w^T for bfloat16 x and w on tcgen05 (see csrc/gemm_tcgen05.cu).  More than
    128 rows go to the kernel that works on pairs of SMs unless ``one_block`` is set."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, out.dtype, "out", contiguous=False)
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue == EPI_GEGLU else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_tcgen05: shapes do not fit")
    entry = library().sib_gemm_tcgen05_one_block if one_block else library().sib_gemm_tcgen05
    _check(entry(_ptr(w), _ptr(x), _ptr(out), _code(out.dtype), c_int(R), c_int(N), c_int(K),
                 c_longlong(x.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_float(cap),
                 _stream()))
    return out


def gemm_tcgen05_error(clear: bool = True) -> int:
    """0, or the code left by a block of gemm_tcgen05 whose bounded wait ran out
    (synchronises the device)."""
    torch.cuda.synchronize()
    return int(library().sib_gemm_tcgen05_error(c_int(1 if clear else 0)))


@_timed(lambda logits, *a, **kw: ("sample_rows", _nbytes(logits), 0))
def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                rng_state: Optional[torch.Tensor], out: torch.Tensor,
                rng_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of 32-bit logits; advances each row's generator by one draw.
    ``rng_index[row]`` (int32) says which element of ``rng_state`` a row uses."""
    _want(logits, torch.float32, "logits", contiguous=False)
    _want(out, torch.int32, "out")
    rows, vocab = logits.shape
    if logits.stride(1) != 1 or out.numel() != rows:
        raise KernelError("sample_rows: shapes do not fit")
    if rng_state is not None:
        _want(rng_state, torch.int64, "rng_state")
        if rng_index is None and rng_state.numel() != rows:
            raise KernelError("sample_rows: one generator state per row")
        if rng_index is not None:
            _want(rng_index, torch.int32, "rng_index")
    _check(library().sib_sample_rows(_ptr(logits), c_longlong(logits.stride(0)), c_int(rows),
                                     c_int(vocab), c_float(temperature), c_int(top_k),
                                     c_float(top_p), _ptr(rng_state), _ptr(rng_index), _ptr(out),
                                     _stream()))
    return out


class KernelWatch:
    """The verdicts of kernels whose waits are bounded, brought to the host without a
    synchronisation of their own.

    ``fetch()`` enqueues an asynchronous copy of the device's error words into a pinned
    buffer on the current stream; after the caller's next synchronisation of that stream
    (the read of the sampled tokens, the copy of the logits) ``check()`` looks at the
    buffer and raises :class:`KernelError` naming the kernel and its code if a wait ran
    out, after clearing the word.  The reference logs a failed launch and goes on
    (src/backend/cuda/mod.rs:379-397)."""

    def __init__(self):
        lib = library()
        lib.sib_error_word_name.restype = ctypes.c_char_p
        self.n = int(lib.sib_error_words())
        self.host = torch.zeros(self.n, dtype=torch.int32).pin_memory()
        self.names = [lib.sib_error_word_name(c_int(i)).decode() for i in range(self.n)]
        self.pending = False

    def fetch(self) -> None:
        if library().sib_kernel_errors_fetch(c_void_p(self.host.data_ptr()), _stream()) != 0:
            raise KernelError(library().sib_last_error().decode())
        self.pending = True

    def check(self) -> None:
        """Call after the stream that ``fetch`` ran on has been synchronised."""
        if not self.pending:
            return
        self.pending = False
        words = self.host.tolist()
        bad = [(i, c) for i, c in enumerate(words) if c]
        if not bad:
            return
        for i, _ in bad:
            set_kernel_error(i, 0)
        self.host.zero_()
        raise KernelError("; ".join(
            f"a bounded wait of {self.names[i] or 'kernel %d' % i} ran out (code {c}): "
            f"its output is incomplete" for i, c in bad))


def set_kernel_error(word: int, code: int) -> None:
    """Set a device error word from the host (0 clears it; tests use it to stand for a
    kernel that gave up)."""
    if library().sib_kernel_error_set(c_int(word), c_int(code), _stream()) != 0:
        raise KernelError(library().sib_last_error().decode())


# --------------------------------------------------------------------------
# decode_chain: several dependent few-row steps as one kernel (csrc/decode_chain.cu)

CHAIN_PRODUCT, CHAIN_NORM = 0, 1
EPI_ROPE = 3


class ChainPhase(ctypes.Structure):
    """Mirrors SibChainPhase of csrc/decode_chain.h."""
    _fields_ = [
        ("kind", c_int), ("epi", c_int),
        ("w", c_void_p), ("x", c_void_p), ("y", c_void_p),
        ("N", c_int), ("K", c_int), ("x_stride", c_int), ("y_stride", c_int), ("out_f32", c_int),
        ("cap", c_float),
        ("row_pos", c_void_p), ("row_seq", c_void_p), ("seq_slot", c_void_p), ("seq_end", c_void_p),
        ("inv_freq", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p), ("page_table", c_void_p),
        ("n_heads", c_int), ("n_kv", c_int), ("head_dim", c_int), ("max_pages", c_int),
        ("page_tokens", c_int), ("ring_tokens", c_int),
        ("a", c_void_p), ("post_gain", c_void_p), ("h", c_void_p), ("pre_gain", c_void_p),
        ("out", c_void_p), ("rows", c_void_p),
        ("post_eps", c_float), ("pre_eps", c_float),
        ("hidden", c_int), ("a_stride", c_int), ("out_stride", c_int),
    ]


def _addr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def chain_product(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                  cap: float = 0.0, rope: Optional[dict] = None) -> ChainPhase:
    """A product phase: out = epilogue(x . w^T).  ``rope``: the arguments of
    ``skinny_linear_rope`` by name, for the q|k|v product that rotates and stores."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue == EPI_GEGLU else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("chain_product: shapes do not fit")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("chain_product: outputs are bfloat16 or float32")
    ph = ChainPhase(kind=CHAIN_PRODUCT, epi=EPI_ROPE if rope is not None else epilogue,
                    w=w.data_ptr(), x=x.data_ptr(), y=out.data_ptr(), N=N, K=K,
                    x_stride=x.stride(0), y_stride=out.stride(0),
                    out_f32=1 if out.dtype == torch.float32 else 0, cap=cap)
    if rope is not None:
        n_kv = rope["n_kv"]
        for name in ("row_pos", "row_seq", "seq_slot", "seq_end"):
            _want(rope[name], torch.int32, name)
            setattr(ph, name, rope[name].data_ptr())
        _want(rope["inv_freq"], torch.float32, "inv_freq")
        if rope["inv_freq"].numel() * 2 != rope["head_dim"]:
            raise KernelError("chain_product: one frequency per pair of the whole head")
        ph.inv_freq = rope["inv_freq"].data_ptr()
        if n_kv:
            _want(rope["k_pool"], torch.bfloat16, "k_pool")
            _want(rope["v_pool"], torch.bfloat16, "v_pool")
            _want(rope["page_table"], torch.int32, "page_table")
            if tuple(rope["k_pool"].shape[1:]) != (n_kv, rope["page_tokens"], rope["head_dim"]):
                raise KernelError("chain_product: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
            ph.k_pool, ph.v_pool = rope["k_pool"].data_ptr(), rope["v_pool"].data_ptr()
            ph.page_table = rope["page_table"].data_ptr()
            ph.max_pages = rope["page_table"].shape[1]
        ph.n_heads, ph.n_kv, ph.head_dim = rope["n_heads"], n_kv, rope["head_dim"]
        ph.page_tokens, ph.ring_tokens = rope["page_tokens"], rope["ring_tokens"]
    return ph


def chain_norm(a: Optional[torch.Tensor], post_gain: Optional[torch.Tensor], post_eps: float,
               h: torch.Tensor, pre_gain: Optional[torch.Tensor], pre_eps: float,
               out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None) -> ChainPhase:
    """A "norm, add, norm" phase (see ``add_rms_norm``); without ``a`` a plain norm of the
    rows of h that ``rows`` names."""
    _want(h, torch.float32, "h")
    hidden = h.shape[1]
    if a is not None:
        _want(a, torch.bfloat16, "a", contiguous=False)
        if tuple(a.shape) != tuple(h.shape) or a.stride(1) != 1:
            raise KernelError("chain_norm: a and h differ in shape")
    for gname, gt in (("post_gain", post_gain), ("pre_gain", pre_gain)):
        if gt is not None:
            _want(gt, torch.float32, gname)
            if gt.numel() != hidden:
                raise KernelError(f"chain_norm: {gname} has the wrong length")
    if pre_gain is not None:
        if out is None:
            raise KernelError("chain_norm: pre_gain needs out")
        _want(out, torch.bfloat16, "out", contiguous=False)
    if rows is not None:
        _want(rows, torch.int32, "rows")
    return ChainPhase(kind=CHAIN_NORM, a=_addr(a), post_gain=_addr(post_gain), h=h.data_ptr(),
                      pre_gain=_addr(pre_gain), out=_addr(out), rows=_addr(rows),
                      post_eps=post_eps, pre_eps=pre_eps, hidden=hidden,
                      a_stride=a.stride(0) if a is not None else 0,
                      out_stride=out.stride(0) if out is not None else 0)


def decode_chain_max_phases() -> int:
    return int(library().sib_decode_chain_max_phases())


def _chain_work(phases, rows, sync, stages=0):
    nbytes = flops = 0
    for ph in phases:
        if ph.kind == CHAIN_PRODUCT:
            nbytes += ph.N * ph.K * 2 + rows * (ph.K + ph.N) * 2
            flops += 2.0 * rows * ph.N * ph.K
        else:
            nbytes += rows * ph.hidden * 12
    return f"decode_chain of {len(phases)}", nbytes, flops


@_timed(_chain_work)
def _decode_chain(phases, rows, sync, stages=0):
    arr = (ChainPhase * len(phases))(*phases)
    _check(library().sib_decode_chain(arr, c_int(len(phases)), c_int(rows), c_int(stages),
                                      _ptr(sync), _stream()))


def decode_chain(phases, rows: int, sync: torch.Tensor, stages: int = 0) -> None:
    """Run ``phases`` (from ``chain_product`` / ``chain_norm``) in order as one kernel for a
    step of ``rows`` rows.  ``sync``: two int32 counters on the device, zero before the
    first call (every call leaves them zero)."""
    _want(sync, torch.int32, "sync")
    if sync.numel() < 2:
        raise KernelError("decode_chain: two counters are needed")
    _decode_chain(list(phases), rows, sync, stages)
