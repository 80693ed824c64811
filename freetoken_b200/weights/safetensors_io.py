"""Reader and writer for the safetensors container, without the safetensors package.

Layout: 8 bytes little-endian header length ``N``; ``N`` bytes of JSON mapping each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative
to the end of the header) plus an optional ``"__metadata__"``; then the raw
little-endian tensor bytes.  Tensors are read by name straight out of a memory map,
as the reference's shard reader does with ``safe_open``
(python/freetoken/models/minimax_m3/weight.py:66-97).  A folder with several shards is
resolved through ``model.safetensors.index.json`` when present, else from the headers
of every ``*.safetensors`` file (python/freetoken/models/weight.py:96-108).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from ..errors import WeightError

_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One ``.safetensors`` file opened for reading by tensor name."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightError(f"{path}: cannot open ({e})") from e
        head = self._f.read(8)
        if len(head) != 8:
            raise WeightError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = os.fstat(self._f.fileno()).st_size
        if n > size - 8:
            raise WeightError(f"{path}: header length {n} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"{path}: header is not valid JSON ({e})") from e
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, dict] = header
        self._base = 8 + n
        self._size = size
        self._map: Optional[mmap.mmap] = None

    def names(self) -> List[str]:
        return list(self.entries.keys())

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        code = self.entries[name]["dtype"]
        if code not in _DTYPES:
            raise WeightError(f"{self.path}: tensor '{name}' has unsupported dtype {code}")
        return _DTYPES[code]

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a view of the file's memory map (copy-on-write, never written back)."""
        e = self.entries[name]
        dtype = self.dtype(name)
        shape = tuple(e["shape"])
        begin, end = e["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        itemsize = torch.empty((), dtype=dtype).element_size()
        if end - begin != count * itemsize or self._base + end > self._size:
            raise WeightError(
                f"{self.path}: tensor '{name}' claims bytes [{begin},{end}) for shape {list(shape)} {e['dtype']}"
            )
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        if self._map is None:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY)
        t = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._base + begin)
        return t.view(shape)

    def close(self) -> None:
        # tensors handed out keep the map alive through the buffer protocol
        self._f.close()


class ModelFolder:
    """All tensors of a model folder, by name, across shards."""

    def __init__(self, folder: str):
        self.folder = folder
        if not os.path.isdir(folder):
            raise WeightError(f"{folder}: not a folder")
        index = os.path.join(folder, "model.safetensors.index.json")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            for name, shard in weight_map.items():
                self._where[name] = shard
        else:
            shards = sorted(x for x in os.listdir(folder) if x.endswith(".safetensors"))
            if not shards:
                raise WeightError(f"{folder}: no .safetensors file in the model folder")
            for shard in shards:
                for name in self._file(shard).names():
                    self._where[name] = shard

    def _file(self, shard: str) -> SafetensorsFile:
        if shard not in self._files:
            self._files[shard] = SafetensorsFile(os.path.join(self.folder, shard))
        return self._files[shard]

    def names(self) -> List[str]:
        return list(self._where.keys())

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._file(self._where[name]).shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._file(self._where[name]).dtype(name)

    def read(self, name: str) -> torch.Tensor:
        return self._file(self._where[name]).read(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write ``tensors`` (CPU, contiguous or not) as one safetensors file."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors.keys())
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write((t if t.dim() else t.reshape(1)).view(torch.uint8).numpy().data)
    os.replace(tmp, path)
