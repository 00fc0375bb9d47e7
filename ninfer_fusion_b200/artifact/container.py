"""`.ninfer` version-2 container: writer, reader and validation.

File = 16-byte prefix (`NINFER\\0\\2` + little-endian u64 JSON length) + UTF-8 JSON directory +
zero padding to a 4096-byte boundary + payloads.  The JSON root has exactly `identity`
(`model_id`, `weights_id`) and `objects`; tensor objects carry exactly
`name, kind, shape, format, layout, offset, bytes`, resource objects exactly
`name, kind, encoding, offset, bytes`; member sets are closed, offsets are relative to the payload
boundary, objects are ordered, aligned and non-overlapping, and a tensor's `bytes` equals its
layout's encoded size (reference: docs/maintainer/artifact-container.md:11-260).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass, field
from typing import BinaryIO, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from . import layouts as L

MAGIC = b"NINFER\x00\x02"
PREFIX_BYTES = 16
PAYLOAD_ALIGNMENT = 4096

FRONTEND_RESOURCES = ("frontend/tokenizer.json", "frontend/tokenizer_config.json", "frontend/chat_template.jinja",
                      "frontend/generation_config.json", "frontend/preprocessor_config.json",
                      "frontend/video_preprocessor_config.json")


class ArtifactError(ValueError):
    pass


@dataclass(frozen=True)
class ArtifactObject:
    name: str
    kind: str                      # "tensor" | "resource"
    offset: int
    bytes: int
    shape: Tuple[int, ...] = ()
    format: str = ""
    layout: str = ""
    encoding: str = ""

    def to_json(self) -> dict:
        if self.kind == "tensor":
            return {"name": self.name, "kind": "tensor", "shape": list(self.shape), "format": self.format,
                    "layout": self.layout, "offset": self.offset, "bytes": self.bytes}
        return {"name": self.name, "kind": "resource", "encoding": self.encoding, "offset": self.offset,
                "bytes": self.bytes}

    @property
    def alignment(self) -> int:
        return L.OBJECT_ALIGNMENT if self.kind == "tensor" else 1


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _exact_members(obj, members: Sequence[str], what: str) -> None:
    if not isinstance(obj, dict):
        raise ArtifactError(f"{what} must be a JSON object")
    if set(obj) != set(members):
        raise ArtifactError(f"{what} must have exactly the members {sorted(members)}, got {sorted(obj)}")


def parse_directory(doc) -> Tuple[Tuple[str, str], List[ArtifactObject]]:
    """Validate a decoded JSON directory against the closed schema."""
    _exact_members(doc, ("identity", "objects"), "root")
    ident = doc["identity"]
    _exact_members(ident, ("model_id", "weights_id"), "identity")
    for k in ("model_id", "weights_id"):
        if not isinstance(ident[k], str) or not ident[k]:
            raise ArtifactError(f"identity.{k} must be a nonempty string")
    objs = doc["objects"]
    if not isinstance(objs, list) or not objs:
        raise ArtifactError("objects must be a nonempty array")
    out: List[ArtifactObject] = []
    names = set()
    cursor = 0
    for i, o in enumerate(objs):
        if not isinstance(o, dict) or o.get("kind") not in ("tensor", "resource"):
            raise ArtifactError(f"object {i}: kind must be 'tensor' or 'resource'")
        if o["kind"] == "tensor":
            _exact_members(o, ("name", "kind", "shape", "format", "layout", "offset", "bytes"), f"tensor object {i}")
            shape = o["shape"]
            if not isinstance(shape, list) or any(not _is_int(d) or d <= 0 for d in shape):
                raise ArtifactError(f"object {i}: shape must be an array of positive integers")
            if o["format"] not in L.FORMATS or o["layout"] not in L.LAYOUTS:
                raise ArtifactError(f"object {i}: unregistered format/layout {o['format']}/{o['layout']}")
            try:
                need = L.encoded_size(o["format"], o["layout"], shape)
            except ValueError as e:
                raise ArtifactError(f"object {i}: {e}") from None
            obj = ArtifactObject(o["name"], "tensor", o["offset"], o["bytes"], tuple(shape), o["format"], o["layout"])
        else:
            _exact_members(o, ("name", "kind", "encoding", "offset", "bytes"), f"resource object {i}")
            if o["encoding"] not in L.ENCODINGS:
                raise ArtifactError(f"object {i}: unregistered encoding {o['encoding']}")
            need = None
            obj = ArtifactObject(o["name"], "resource", o["offset"], o["bytes"], encoding=o["encoding"])
        if not isinstance(obj.name, str) or not obj.name:
            raise ArtifactError(f"object {i}: name must be a nonempty string")
        if obj.name in names:
            raise ArtifactError(f"duplicate object name {obj.name}")
        names.add(obj.name)
        if not _is_int(obj.offset) or obj.offset < 0 or not _is_int(obj.bytes) or obj.bytes <= 0:
            raise ArtifactError(f"object {obj.name}: offset must be >= 0 and bytes > 0")
        if need is not None and need != obj.bytes:
            raise ArtifactError(f"object {obj.name}: bytes {obj.bytes} != encoded size {need}")
        if obj.offset % obj.alignment:
            raise ArtifactError(f"object {obj.name} is not {obj.alignment}-byte aligned")
        if obj.offset < cursor:
            raise ArtifactError(f"object {obj.name} overlaps or precedes the previous object")
        cursor = obj.offset + obj.bytes
        out.append(obj)
    return (ident["model_id"], ident["weights_id"]), out


class ArtifactWriter:
    """Streams an artifact to disk: `add_*` collects the inventory, `write` lays it out and emits it."""

    def __init__(self, model_id: str, weights_id: str):
        self.identity = (model_id, weights_id)
        self._items: List[Tuple[dict, bytes]] = []

    def add_tensor(self, name: str, tensor: torch.Tensor, fmt: str = "BF16") -> None:
        payload, layout = L.encode_tensor(tensor, fmt)
        self._items.append(({"name": name, "kind": "tensor", "shape": list(tensor.shape), "format": fmt,
                             "layout": layout}, payload))

    def add_encoded(self, name: str, shape: Sequence[int], fmt: str, layout: str, payload: bytes) -> None:
        if len(payload) != L.encoded_size(fmt, layout, shape):
            raise ArtifactError(f"{name}: payload length does not match the encoded size")
        self._items.append(({"name": name, "kind": "tensor", "shape": list(shape), "format": fmt, "layout": layout},
                            payload))

    def add_resource(self, name: str, data: bytes) -> None:
        if not data:
            raise ArtifactError("a resource must not be empty")
        self._items.append(({"name": name, "kind": "resource", "encoding": "raw-bytes-v1"}, data))

    def write(self, path: str) -> None:
        cursor = 0
        objects = []
        for meta, payload in self._items:
            align = L.OBJECT_ALIGNMENT if meta["kind"] == "tensor" else 1
            cursor = L.align_up(cursor, align)
            objects.append(dict(meta, offset=cursor, bytes=len(payload)))
            cursor += len(payload)
        doc = {"identity": {"model_id": self.identity[0], "weights_id": self.identity[1]}, "objects": objects}
        parse_directory(doc)
        text = json.dumps(doc, separators=(",", ":")).encode("utf-8")
        payload_offset = L.align_up(PREFIX_BYTES + len(text), PAYLOAD_ALIGNMENT)
        with open(path, "wb") as f:
            f.write(MAGIC + struct.pack("<Q", len(text)))
            f.write(text)
            f.write(bytes(payload_offset - PREFIX_BYTES - len(text)))
            pos = 0
            for o, (_, payload) in zip(objects, self._items):
                if o["offset"] > pos:
                    f.write(bytes(o["offset"] - pos))
                f.write(payload)
                pos = o["offset"] + len(payload)


class ArtifactReader:
    """mmap-backed reader with full directory validation (pure Python twin of the native reader)."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        head = self._f.read(PREFIX_BYTES)
        if len(head) != PREFIX_BYTES or head[:8] != MAGIC:
            raise ArtifactError("not a .ninfer version-2 artifact (bad magic)")
        (json_bytes,) = struct.unpack("<Q", head[8:])
        if json_bytes <= 0 or PREFIX_BYTES + json_bytes > size:
            raise ArtifactError("declared JSON range lies outside the file")
        text = self._f.read(json_bytes)
        try:
            doc = json.loads(text.decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise ArtifactError(f"directory is not valid UTF-8 JSON: {e}") from None
        self.identity, self.objects = parse_directory(doc)
        self.payload_offset = L.align_up(PREFIX_BYTES + json_bytes, PAYLOAD_ALIGNMENT)
        if self.payload_offset > size:
            raise ArtifactError("file ends before the payload boundary")
        last = self.objects[-1]
        if self.payload_offset + last.offset + last.bytes > size:
            raise ArtifactError("an object extends past the end of the file")
        self.by_name: Dict[str, ArtifactObject] = {o.name: o for o in self.objects}
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def close(self) -> None:
        self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def payload(self, name: str) -> memoryview:
        o = self.by_name[name]
        start = self.payload_offset + o.offset
        return memoryview(self._mm)[start:start + o.bytes]

    def resource(self, name: str) -> bytes:
        o = self.by_name[name]
        if o.kind != "resource":
            raise ArtifactError(f"{name} is not a resource")
        return bytes(self.payload(name))

    def tensor(self, name: str) -> torch.Tensor:
        """Represented values (direct formats keep their dtype, quantised formats decode to fp32)."""
        o = self.by_name[name]
        if o.kind != "tensor":
            raise ArtifactError(f"{name} is not a tensor")
        return L.decode_tensor(bytes(self.payload(name)), o.format, o.layout, o.shape)

    def tensors(self) -> Iterable[str]:
        return (o.name for o in self.objects if o.kind == "tensor")


def rank_artifact_name(path: str, rank: int, world: int) -> str:
    """Per-rank artifact naming for tensor-parallel shards: `model.tp1of4.ninfer` (reference: src/core/shard_plan.h:276-290)."""
    if world == 1:
        return path
    stem, ext = os.path.splitext(path)
    return f"{stem}.tp{rank}of{world}{ext}"
