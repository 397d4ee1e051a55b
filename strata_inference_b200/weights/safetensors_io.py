"""Reading and writing safetensors files, by tensor name.

File layout: an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` (plus an
optional ``__metadata__`` entry), then the data region the offsets index.
A model folder holds either ``model.safetensors`` or several shards with a
``model.safetensors.index.json`` whose ``weight_map`` names each tensor's file.

The reference fetches tensors by name from its own container format
(src/model/weights.rs:133-193); this module is that fetch for safetensors.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped file; ``get`` returns a tensor that views the map."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size")
        try:
            header = json.loads(self._f.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + hlen
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: Dict[str, dict] = {}
        for name, e in header.items():
            if e.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unknown dtype {e.get('dtype')!r}")
            b, en = e["data_offsets"]
            n = 1
            for s in e["shape"]:
                n *= s
            want = n * torch.empty((), dtype=_DTYPES[e["dtype"]]).element_size()
            if en - b != want or self._data_start + en > size:
                raise SafetensorsError(f"{path}: tensor '{name}' has {en - b} bytes of data, "
                                       f"its shape {e['shape']} needs {want}")
            self.entries[name] = e

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def get(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        b, en = e["data_offsets"]
        dt = _DTYPES[e["dtype"]]
        if en == b:
            return torch.empty(tuple(e["shape"]), dtype=dt)
        buf = memoryview(self._map)[self._data_start + b:self._data_start + en]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; nobody writes through it
            t = torch.frombuffer(buf, dtype=dt)
        return t.view(tuple(e["shape"]))


class ModelFiles:
    """All safetensors files of a model folder, as one name -> tensor table."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.isfile(index):
            with open(index) as f:
                weight_map = json.load(f).get("weight_map", {})
            for fname in sorted(set(weight_map.values())):
                self._files[fname] = SafetensorsFile(os.path.join(model_dir, fname))
            for name, fname in weight_map.items():
                if name not in self._files[fname].entries:
                    raise SafetensorsError(f"{index}: '{name}' is mapped to {fname}, "
                                           f"which does not hold it")
                self._where[name] = fname
        elif os.path.isfile(single):
            sf = SafetensorsFile(single)
            self._files["model.safetensors"] = sf
            for name in sf.names():
                self._where[name] = "model.safetensors"
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor "
                                   f"model.safetensors.index.json found")

    def names(self) -> List[str]:
        return list(self._where)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._files[self._where[name]].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._files[self._where[name]].dtype(name)

    def get(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].get(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] = None) -> None:
    """Write ``tensors`` (CPU or device) to ``path`` in the order given."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((-len(blob)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, t in tensors.items():
            c = t.detach().contiguous().cpu()
            if c.numel():
                f.write(c.view(torch.uint8).numpy().tobytes() if c.dim() else
                        c.reshape(1).view(torch.uint8).numpy().tobytes())
