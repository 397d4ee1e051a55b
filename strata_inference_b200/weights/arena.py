"""The model's weights in ONE device allocation, filled in place.

Parts say what they keep on the device (*resident* tensors) and how each is
put together from *stored* tensors (the ones a model folder holds):

    Resident(shape, dtype, pieces=(Piece("q_proj.weight", row_offset=0), ...))

A piece places the rows of one stored tensor into the resident tensor, either
as one run (``row_offset``) or as runs of ``group`` rows whose starts lie
``group_stride`` resident rows apart (how a gate and an up matrix are
interleaved).  ``offset`` is added to every element (a norm's ``1 + weight``).
``dtype`` is a torch type, ``COMPUTE`` (the engine's compute type) or
``STORED`` (the type the source keeps the tensor in).

``WeightArena`` lays every resident tensor out in one buffer (256-byte aligned
sub-buffers) and a *source* writes the pieces straight to their places: from
the mapped file in bounded chunks (``FileSource``), from tensors in memory
(``DictSource``) or from the seeded generator on the device
(``RandomSource``).  Nothing is concatenated or re-laid-out beside the arena,
so loading needs the weights' own bytes plus one chunk.

The reference allocates every tensor on its own (src/backend/cuda/mod.rs:264-276)
and splits fused tensors on the host (src/model/weights.rs:219-289, 335-399); this
model wants the opposite direction (separate stored tensors, fused resident ones).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional, Tuple, Union

import torch

from .loader import TensorDecl, storage_dtype

COMPUTE = "compute"
STORED = "stored"
_ALIGN = 256
_CHUNK_BYTES = 32 << 20


@dataclass(frozen=True)
class Piece:
    source: str              # local name of the stored tensor
    row_offset: int = 0      # resident row of the stored tensor's first row
    group: int = 0           # 0: the rows stay together
    group_stride: int = 0    # with group > 0: resident rows between the starts of two runs


@dataclass(frozen=True)
class Resident:
    shape: Tuple[int, ...]
    dtype: Union[str, torch.dtype] = COMPUTE
    pieces: Tuple[Piece, ...] = ()
    offset: float = 0.0


def resident_of(part_class, stored: Mapping[str, TensorDecl], *args) -> Dict[str, Resident]:
    """What a part keeps on the device: its own ``resident(...)`` declaration if it
    has one, else every stored tensor as it is stored, under the same name."""
    if hasattr(part_class, "resident"):
        return dict(part_class.resident(*args))
    return {name: Resident(tuple(d.shape), STORED, (Piece(name),))
            for name, d in stored.items()}


def _rows_cols(shape: Tuple[int, ...]) -> Tuple[int, int]:
    if len(shape) == 0:
        return 1, 1
    cols = 1
    for s in shape[1:]:
        cols *= int(s)
    return int(shape[0]), cols


class WeightArena:
    """One buffer, one view per resident tensor.  ``plan``: full resident name ->
    (Resident, prefix of its pieces' stored names)."""

    def __init__(self, plan: Mapping[str, Tuple[Resident, str]], compute_dtype: torch.dtype,
                 device, stored_dtypes: Optional[Mapping[str, torch.dtype]] = None):
        self.plan = dict(plan)
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype
        layout, total = [], 0
        for name, (res, prefix) in self.plan.items():
            dtype = res.dtype
            if dtype == COMPUTE:
                dtype = compute_dtype
            elif dtype == STORED:
                first = prefix + res.pieces[0].source if res.pieces else None
                have = (stored_dtypes or {}).get(first)
                dtype = storage_dtype(have) if have is not None else compute_dtype
            n = 1
            for s in res.shape:
                n *= int(s)
            nbytes = n * torch.empty((), dtype=dtype).element_size()
            layout.append((name, dtype, tuple(res.shape), total, nbytes))
            total += -(-nbytes // _ALIGN) * _ALIGN
        self.nbytes = total
        self.buffer = torch.empty(max(total, _ALIGN), dtype=torch.uint8, device=self.device)
        self.tensors: Dict[str, torch.Tensor] = {}
        for name, dtype, shape, begin, nbytes in layout:
            self.tensors[name] = self.buffer[begin:begin + nbytes].view(dtype).view(shape)

    def fill(self, source) -> "WeightArena":
        for name, (res, prefix) in self.plan.items():
            dst = self.tensors[name]
            rows, cols = _rows_cols(res.shape)
            flat = dst.view(rows, cols)
            for piece in res.pieces:
                source.write(prefix + piece.source, flat, piece, res.offset)
        return self


def _target(flat: torch.Tensor, piece: Piece, rows: int) -> torch.Tensor:
    """The [runs, rows a run, cols] view of ``flat`` that a piece of ``rows`` rows fills."""
    cols = flat.shape[1]
    group = piece.group or rows
    stride = piece.group_stride if piece.group else rows
    if rows % max(group, 1):
        raise ValueError(f"'{piece.source}': {rows} rows are not whole runs of {group}")
    runs = rows // group if group else 0
    last = piece.row_offset + (runs - 1) * stride + group if runs else piece.row_offset
    if last > flat.shape[0]:
        raise ValueError(f"'{piece.source}': its rows end at {last}, the resident tensor "
                         f"has {flat.shape[0]}")
    return flat.as_strided((runs, group, cols), (stride * cols, cols, 1),
                           flat.storage_offset() + piece.row_offset * cols)


class DictSource:
    """Stored tensors in memory (host or device), by full name."""

    def __init__(self, tensors: Mapping[str, torch.Tensor]):
        self.tensors = tensors

    def table(self) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        return {n: (tuple(t.shape), t.dtype) for n, t in self.tensors.items()}

    def read(self, name: str) -> torch.Tensor:
        return self.tensors[name]

    def write(self, name: str, flat: torch.Tensor, piece: Piece, offset: float) -> None:
        src = self.read(name)
        rows, cols = _rows_cols(tuple(src.shape))
        if cols != flat.shape[1]:
            raise ValueError(f"'{name}': rows of {cols} elements do not fit rows of {flat.shape[1]}")
        dst = _target(flat, piece, rows)
        runs, group, _ = dst.shape
        src = src.reshape(runs, group, cols)
        per_run = max(1, group * cols * src.element_size())
        step = max(1, _CHUNK_BYTES // per_run)
        for r0 in range(0, runs, step):
            if runs == 1 and per_run > _CHUNK_BYTES:
                # one long run: cut it by rows instead
                row_step = max(1, _CHUNK_BYTES // max(1, cols * src.element_size()))
                for g0 in range(0, group, row_step):
                    dst[0, g0:g0 + row_step].copy_(src[0, g0:g0 + row_step])
            else:
                dst[r0:r0 + step].copy_(src[r0:r0 + step])
        if offset:
            dst.add_(offset)


class FileSource(DictSource):
    """The safetensors files of a model folder (mapped, read piece by piece)."""

    def __init__(self, files):
        self.files = files

    def table(self):
        return {n: (self.files.shape(n), self.files.dtype(n)) for n in self.files.names()}

    def read(self, name: str) -> torch.Tensor:
        return self.files.get(name)


class RandomSource:
    """Seeded random values (weights/random_init.py), drawn by the device's kernel
    straight into the arena, or on the host when the arena is not on a device."""

    def __init__(self, expected: Mapping[str, TensorDecl], seed: int, stored_dtype: torch.dtype,
                 matrix_std: float, norm_std: float):
        self.expected = expected
        self.seed = seed
        self.stored_dtype = stored_dtype     # what write_random_model would store them in
        self.matrix_std = matrix_std
        self.norm_std = norm_std

    def table(self):
        return {n: (tuple(d.shape), torch.int32 if d.integer else self.stored_dtype)
                for n, d in self.expected.items() if not d.optional}

    def write(self, name: str, flat: torch.Tensor, piece: Piece, offset: float) -> None:
        from .random_init import randn_host, std_of, tensor_key
        decl = self.expected[name]
        rows, cols = _rows_cols(tuple(decl.shape))
        dst = _target(flat, piece, rows)
        if decl.integer:
            dst.zero_()
            return
        std = std_of(decl, self.matrix_std, self.norm_std)
        if flat.is_cuda:
            from ..kernels import native
            native.randn_fill(dst, rows, cols, piece.group, piece.group_stride,
                              tensor_key(self.seed, name), offset, std, self.stored_dtype)
        else:
            host = randn_host(decl.shape, self.seed, name, std, self.stored_dtype).float()
            dst.copy_((host + offset if offset else host).reshape(dst.shape))
