"""Reader and writer for the safetensors container (no third-party package).

Layout of a file: 8 bytes little-endian header length ``n``; ``n`` bytes of JSON
mapping each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}``
(offsets relative to the end of the header; an optional ``"__metadata__"`` entry);
then the raw little-endian tensor bytes.  A folder may hold one
``model.safetensors`` or shards listed by ``model.safetensors.index.json``
(``{"weight_map": {tensor name: file name}}``).

The reference never opens these files itself (it goes through a library loader,
engine/engine.py:184-207); tensor names are the ones that loader's module tree
implies (OPTIMIZATION_GUIDE.md:116-131).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors container."""


# safetensors dtype tag -> (torch dtype, numpy carrier dtype, bytes per element)
_DTYPES = {
    "F64": (torch.float64, np.dtype("<f8"), 8),
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "BF16": (torch.bfloat16, np.dtype("<u2"), 2),
    "I64": (torch.int64, np.dtype("<i8"), 8),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I16": (torch.int16, np.dtype("<i2"), 2),
    "I8": (torch.int8, np.dtype("i1"), 1),
    "U8": (torch.uint8, np.dtype("u1"), 1),
    "BOOL": (torch.bool, np.dtype("u1"), 1),
}
_TAG_OF = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    path: str
    begin: int  # absolute byte offsets in the file
    end: int


class SafetensorsFile:
    """One opened file: the parsed header, and tensors read on demand from a map."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError:
            raise SafetensorsError(f"{path}: not found") from None
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (only {size} bytes, no header length)")
        with open(path, "rb") as handle:
            (n,) = struct.unpack("<Q", handle.read(8))
            if n > size - 8:
                raise SafetensorsError(f"{path}: header length {n} exceeds file size {size}")
            raw = handle.read(n)
        try:
            header = json.loads(raw.decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{path}: header is not valid JSON ({error})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        base = 8 + n
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                tag, shape, (begin, end) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for '{name}'") from None
            if tag not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unknown dtype '{tag}'")
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if end - begin != count * _DTYPES[tag][2]:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' {tag}{list(shape)} needs {count * _DTYPES[tag][2]} bytes, "
                    f"header gives {end - begin}")
            if begin < 0 or base + end > size:
                raise SafetensorsError(
                    f"{path}: truncated: tensor '{name}' ends at byte {base + end}, file has {size}")
            self.entries[name] = TensorEntry(name, _DTYPES[tag][0], shape, path, base + begin, base + end)
        self._map = None

    def _buffer(self):
        if self._map is None:
            with open(self.path, "rb") as handle:
                self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ)
        return self._map

    def read(self, name: str) -> torch.Tensor:
        """The tensor in its stored dtype, as a fresh CPU tensor."""
        entry = self.entries[name]
        tag = _TAG_OF[entry.dtype]
        carrier = _DTYPES[tag][1]
        array = np.frombuffer(self._buffer(), dtype=carrier, count=(entry.end - entry.begin) // carrier.itemsize,
                              offset=entry.begin).copy()
        tensor = torch.from_numpy(array)
        if entry.dtype == torch.bfloat16:
            tensor = tensor.view(torch.int16).view(torch.bfloat16)
        elif entry.dtype == torch.bool:
            tensor = tensor.to(torch.bool)
        return tensor.reshape(entry.shape)


class Checkpoint:
    """All tensors of a model folder, whichever file holds them."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self.files: Dict[str, SafetensorsFile] = {}
        self.entries: Dict[str, TensorEntry] = {}
        if os.path.exists(index):
            with open(index) as handle:
                weight_map = json.load(handle).get("weight_map", {})
            for name, file_name in weight_map.items():
                path = os.path.join(model_dir, file_name)
                if path not in self.files:
                    self.files[path] = SafetensorsFile(path)
                if name not in self.files[path].entries:
                    raise SafetensorsError(f"{index}: lists '{name}' in {file_name}, which does not hold it")
            for f in self.files.values():
                self.entries.update(f.entries)
        elif os.path.exists(single):
            self.files[single] = SafetensorsFile(single)
            self.entries.update(self.files[single].entries)
        else:
            raise SafetensorsError(
                f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def read(self, name: str) -> torch.Tensor:
        return self.files[self.entries[name].path].read(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write tensors (CPU, any listed dtype) in the order given."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    blobs = []
    for name, tensor in tensors.items():
        if tensor.dtype not in _TAG_OF:
            raise SafetensorsError(f"tensor '{name}': dtype {tensor.dtype} cannot be stored")
        t = tensor.detach().contiguous().cpu()
        if t.dtype == torch.bfloat16:
            data = t.view(torch.int16).numpy().tobytes()
        elif t.dtype == torch.bool:
            data = t.to(torch.uint8).numpy().tobytes()
        else:
            data = t.numpy().tobytes()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(data)]}
        offset += len(data)
        blobs.append(data)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(raw)))
        handle.write(raw)
        for data in blobs:
            handle.write(data)
