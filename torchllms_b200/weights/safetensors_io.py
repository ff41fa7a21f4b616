"""Reading and writing safetensors files by tensor name.

The reference converts Hugging Face checkpoints offline into a pickled
``consolidated.00.pth`` (torchllms/models/checkpoint_converter.py:70-78,
:271-346) and loads that with ``torch.load(mmap=True)``
(torchllms/models/utils.py:96-111).  This engine reads safetensors directly:
an 8-byte little-endian header length, a JSON header
``{name: {dtype, shape, data_offsets}}`` and the raw data, which is mapped
into memory so that only the tensors that are asked for are touched.  A
folder may hold one ``model.safetensors`` or shards listed in
``model.safetensors.index.json`` (``weight_map``: name -> file), the discovery
order of torchllms/models/checkpoint_converter.py:276-307.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Dict, Iterable, Iterator, List, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One file, mapped; ``get(name)`` returns a CPU tensor that views the map."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
        with open(self.path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            if n > size - 8:
                raise SafetensorsError(f"{self.path}: header length {n} exceeds the file size")
            try:
                header = json.loads(f.read(n).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{self.path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._entries: Dict[str, dict] = header
        self._data_start = 8 + n
        self._data_len = size - self._data_start
        self._map = None
        for name, e in header.items():
            if e.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {e.get('dtype')!r}")
            lo, hi = e["data_offsets"]
            count = int(np.prod(e["shape"], dtype=np.int64)) if e["shape"] else 1
            width = torch.empty((), dtype=_DTYPES[e["dtype"]]).element_size()
            if not (0 <= lo <= hi <= self._data_len) or hi - lo != count * width:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has inconsistent offsets {lo}:{hi}")

    def names(self) -> List[str]:
        return list(self._entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self._entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._entries[name]["dtype"]]

    def get(self, name: str) -> torch.Tensor:
        e = self._entries[name]
        lo, hi = e["data_offsets"]
        dtype = _DTYPES[e["dtype"]]
        shape = tuple(e["shape"])
        if hi == lo:
            return torch.empty(shape, dtype=dtype)
        if self._map is None:
            # copy-on-write mapping: pages are read lazily and torch sees a writable buffer
            self._map = np.memmap(self.path, dtype=np.uint8, mode="c", offset=self._data_start,
                                  shape=(self._data_len,))
        raw = torch.from_numpy(self._map[lo:hi])
        if dtype == torch.bool:
            return raw.view(torch.uint8).reshape(shape).to(torch.bool)
        return raw.view(dtype).reshape(shape)


class TorchCheckpointFile:
    """A ``torch.save``d dictionary of tensors (the reference's ``consolidated.00.pth``, which it
    reads with ``torch.load(mmap=True)``, torchllms/models/utils.py:107-111), offered by name like a
    safetensors file.  Only tensors are unpickled (``weights_only``); the file is mapped, not read."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            state = torch.load(str(self.path), mmap=True, weights_only=True, map_location="cpu")
        except Exception as e:          # a pickle that holds more than tensors, a truncated file, ...
            raise SafetensorsError(f"{self.path}: not a checkpoint of plain tensors ({type(e).__name__}: {e})") from None
        if not isinstance(state, dict) or not all(isinstance(k, str) and isinstance(v, torch.Tensor) for k, v in state.items()):
            raise SafetensorsError(f"{self.path}: expected a dictionary from tensor names to tensors")
        self._state = state

    def names(self) -> List[str]:
        return list(self._state)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self._state[name].shape)

    def dtype(self, name: str) -> torch.dtype:
        return self._state[name].dtype

    def get(self, name: str) -> torch.Tensor:
        return self._state[name]


TORCH_SUFFIXES = (".pth", ".pt")


class TensorSource:
    """All tensors of a model folder (or a single file), by name: safetensors (one file, or shards
    with their index), or, where a folder holds none, the reference's ``consolidated.*.pth``."""

    def __init__(self, path):
        path = Path(path)
        self.files: List[SafetensorsFile] = []
        self._where: Dict[str, SafetensorsFile] = {}
        if path.is_file():
            paths = [path]
        else:
            index = path / "model.safetensors.index.json"
            single = path / "model.safetensors"
            if index.is_file():
                with open(index) as f:
                    weight_map = json.load(f).get("weight_map", {})
                paths = [path / name for name in sorted(set(weight_map.values()))]
            elif single.is_file():
                paths = [single]
            else:
                paths = sorted(path.glob("*.safetensors")) or sorted(path.glob("consolidated.*.pth"))
            if not paths:
                raise FileNotFoundError(f"{path}: no model.safetensors (or shards, or consolidated.*.pth) found")
        for p in paths:
            if not p.is_file():
                raise FileNotFoundError(f"{p}: listed in the shard index but missing")
            f = TorchCheckpointFile(p) if p.suffix in TORCH_SUFFIXES else SafetensorsFile(p)
            self.files.append(f)
            for name in f.names():
                if name in self._where:
                    raise SafetensorsError(f"tensor {name!r} appears in both {self._where[name].path} and {p}")
                self._where[name] = f

    def names(self) -> List[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def get(self, name: str) -> torch.Tensor:
        return self._where[name].get(name)

    def items(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for name in self._where:
            yield name, self.get(name)


def write_safetensors(path, tensors: Iterable[Tuple[str, torch.Tensor]] | Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] | None = None) -> None:
    """Write tensors (CPU, any supported dtype) to one safetensors file."""
    if isinstance(tensors, Mapping):
        tensors = tensors.items()
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs: List[Tuple[torch.Tensor, int]] = []
    offset = 0
    for name, t in tensors:
        if name in header:
            raise SafetensorsError(f"tensor {name!r} given twice")
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        t = t.detach().to("cpu").contiguous()
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        blobs.append((t, nbytes))
        offset += nbytes
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * ((8 - len(head) % 8) % 8)
    path = Path(path)
    tmp = path.with_name(path.name + ".tmp")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for t, nbytes in blobs:
            if nbytes:
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    tmp.replace(path)
