"""A small reader and writer for the safetensors container.

Layout: 8 bytes little-endian header length, a JSON header that maps each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), then the raw little-endian tensor bytes.
A folder may hold one ``model.safetensors`` or several shards listed in
``model.safetensors.index.json`` under ``weight_map``.  The reference reads a
different container (GGUF, crates/leone-gguf/src/container.rs); what is kept
from it is the strictness: every offset and size is checked before use.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    file: str
    begin: int      # absolute byte offset in the file
    nbytes: int


class SafetensorsFile:
    """One open ``.safetensors`` file; tensors are read lazily from a memory map."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8 or hlen > (100 << 20):
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as err:
            raise SafetensorsError(f"{path}: header is not valid JSON ({err})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        data_start = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype_name = meta["dtype"]
                shape = tuple(int(s) for s in meta["shape"])
                begin, end = (int(x) for x in meta["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}'") from None
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype_name}")
            dtype, width = _DTYPES[dtype_name]
            count = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor '{name}' has a negative dimension")
                count *= s
            if end - begin != count * width or begin < 0 or data_start + end > size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' byte range [{begin},{end}) does not match "
                    f"shape {list(shape)} of {dtype_name} or leaves the file")
            self.entries[name] = TensorEntry(name, dtype, shape, path, data_start + begin, end - begin)
        self._map = None

    def _mapping(self):
        if self._map is None:
            self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        return self._map

    def read(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e.nbytes == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._mapping())[e.begin:e.begin + e.nbytes]
        # A copy detaches the tensor from the map so the file can be closed.
        flat = torch.frombuffer(bytearray(buf), dtype=e.dtype)
        return flat.reshape(e.shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._fh.close()


class Checkpoint:
    """All tensors of a model folder, whichever shard holds them."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        files: List[str] = []
        if os.path.isfile(index):
            with open(index) as fh:
                weight_map = json.load(fh).get("weight_map", {})
            files = sorted({os.path.join(folder, f) for f in weight_map.values()})
        elif os.path.isfile(single):
            files = [single]
        else:
            raise SafetensorsError(f"{folder}: no model.safetensors (or index) found")
        self.files = [SafetensorsFile(f) for f in files]
        self.entries: Dict[str, TensorEntry] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name, entry in f.entries.items():
                if name in self.entries:
                    raise SafetensorsError(f"tensor '{name}' appears in two shards")
                self.entries[name] = entry
                self._owner[name] = f

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def read(self, name: str) -> torch.Tensor:
        return self._owner[name].read(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            fh.write(t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b"")
