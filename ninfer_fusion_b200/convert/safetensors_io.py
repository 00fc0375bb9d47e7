"""Minimal safetensors reader / writer (no dependency on the safetensors package).

File layout: u64 little-endian header length, a JSON header {name: {dtype, shape, data_offsets: [begin, end]}},
then the raw little-endian tensor bytes.  Tensors are read lazily through a memory map, one at a time, so a
checkpoint far larger than host memory can be converted leaf by leaf.
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > 256 << 20:
            raise ValueError(f"{path}: implausible safetensors header ({n} bytes)")
        self.header: Dict[str, dict] = json.loads(self._f.read(n).decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def names(self) -> List[str]:
        return list(self.header)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.header[name]["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        e = self.header[name]
        dt = _DTYPES.get(e["dtype"])
        if dt is None:
            raise ValueError(f"{self.path}: tensor {name} has unsupported dtype {e['dtype']}")
        b, end = e["data_offsets"]
        buf = memoryview(self._mm)[self._base + b: self._base + end]
        t = torch.frombuffer(bytearray(buf), dtype=torch.uint8).view(dt)   # private writable copy of this tensor only
        return t.view(tuple(e["shape"]))

    def close(self) -> None:
        self._mm.close()
        self._f.close()


class SafetensorsSource:
    """All tensors of a checkpoint directory (sharded or single file), looked up by name."""

    def __init__(self, path: str):
        files: List[str]
        if os.path.isdir(path):
            index = os.path.join(path, "model.safetensors.index.json")
            if os.path.exists(index):
                with open(index, encoding="utf-8") as f:
                    wm = json.load(f)["weight_map"]
                files = sorted({os.path.join(path, v) for v in wm.values()})
            else:
                files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
        else:
            files = [path]
        if not files:
            raise FileNotFoundError(f"no safetensors files under {path}")
        self.files = [SafetensorsFile(f) for f in files]
        self.where: Dict[str, SafetensorsFile] = {}
        for sf in self.files:
            for n in sf.names():
                self.where[n] = sf

    def __contains__(self, name: str) -> bool:
        return name in self.where

    def names(self) -> List[str]:
        return list(self.where)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.where[name].shape(name)

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self.where:
            raise KeyError(f"checkpoint has no tensor '{name}'")
        return self.where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    header: Dict[str, dict] = {}
    off = 0
    items: List[Tuple[str, torch.Tensor]] = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"{name}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
        items.append((name, t))
    if metadata:
        header["__metadata__"] = dict(metadata)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
