"""Reading and writing safetensors files by tensor name.

File layout (src/format/safetensors.zig:5-9,213-227): an unsigned 64-bit
little-endian header length n, n bytes of JSON mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` with offsets relative to
byte 8 + n, then the data.  A folder holds one ``model.safetensors`` or
several shards named by ``model.safetensors.index.json``'s ``weight_map``;
without an index every ``*.safetensors`` file is read in name order
(src/format/safetensors.zig:117-168,1345-1384).

Every offset and size is checked when the file is opened
(src/format/safetensors.zig:18-30,360-406), so a truncated or inconsistent
file fails there and not in a kernel.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024       # src/format/safetensors.zig:18-30

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int          # absolute byte offsets in the file
    end: int
    path: str


class SafetensorsFile:
    """One shard, memory-mapped; tensors are views until copied."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte header length")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > MAX_HEADER_BYTES or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file or the "
                                   f"{MAX_HEADER_BYTES}-byte limit")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        base = 8 + n
        self.metadata = header.pop("__metadata__", None)
        self.tensors: Dict[str, TensorInfo] = {}
        for name, e in header.items():
            try:
                dtype, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}'") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype}")
            numel = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor '{name}' has a negative dimension")
                numel *= s
            if en < b or en - b != numel * _DTYPES[dtype][1]:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' spans {en - b} bytes but shape {list(shape)} "
                    f"of {dtype} needs {numel * _DTYPES[dtype][1]}")
            if base + en > size:
                raise SafetensorsError(f"{path}: tensor '{name}' ends beyond the file")
            self.tensors[name] = TensorInfo(name, dtype, shape, base + b, base + en, path)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped bytes (read-only: clone before writing)."""
        info = self.tensors[name]
        dtype, _ = _DTYPES[info.dtype]
        n = info.end - info.begin
        if n == 0:
            return torch.empty(info.shape, dtype=dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # the buffer is read-only on purpose
            flat = torch.frombuffer(self._mm, dtype=dtype, count=n // _DTYPES[info.dtype][1],
                                    offset=info.begin)
        return flat.reshape(info.shape)

    def close(self):
        # tensors handed out keep the map alive through the buffer protocol
        self._f.close()


class SafetensorsFolder:
    """All shards of a model folder behind one name -> tensor view."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        if os.path.isfile(index):
            with open(index, "r") as f:
                wm = json.load(f).get("weight_map", {})
            shard_names: List[str] = []
            for v in wm.values():
                # a shard name must stay inside the folder
                # (src/format/safetensors.zig:1333-1340)
                if os.path.basename(v) != v or v in ("", ".", ".."):
                    raise SafetensorsError(f"{index}: shard name {v!r} leaves the folder")
                if v not in shard_names:
                    shard_names.append(v)
        else:
            shard_names = sorted(n for n in os.listdir(folder) if n.endswith(".safetensors"))
        if not shard_names:
            raise SafetensorsError(f"{folder}: no .safetensors file")
        self.shards: List[SafetensorsFile] = []
        self.tensors: Dict[str, TensorInfo] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        for sn in shard_names:
            p = os.path.join(folder, sn)
            if not os.path.isfile(p):
                raise SafetensorsError(f"{folder}: shard {sn} named by the index is missing")
            sf = SafetensorsFile(p)
            self.shards.append(sf)
            for name, info in sf.tensors.items():
                if name in self.tensors:
                    raise SafetensorsError(f"tensor '{name}' appears in both "
                                           f"{self.tensors[name].path} and {p}")
                self.tensors[name] = info
                self._owner[name] = sf

    def names(self) -> Iterable[str]:
        return self.tensors.keys()

    def tensor(self, name: str) -> torch.Tensor:
        return self._owner[name].tensor(name)


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Write tensors (CPU, contiguous) under their names, in name order."""
    header: Dict[str, dict] = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b"")
