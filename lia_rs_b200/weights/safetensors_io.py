"""A checked little-endian safetensors reader and writer.

Format: 8-byte little-endian header length, a JSON header mapping tensor names to
{dtype, shape, data_offsets}, then the tensor bytes.  The checks are the reference's
(src/safetensors.rs:66-156): header length bounds, extents equal to shape x dtype size,
no gaps or overlaps, no bytes that the header does not index.  A model folder holds either
`model.safetensors` or `model.safetensors.index.json` with a `weight_map` over shards
(src/safetensors/archive.rs:16-86).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    dtype: torch.dtype
    shape: tuple
    start: int      # byte offset inside the data section
    nbytes: int


def parse_header(header: bytes, data_len: int) -> dict:
    """Validate a header against the length of the data section; name -> TensorEntry."""
    if not header or header[:1] != b"{":
        raise SafetensorsError("safetensors header must start with an object")
    try:
        obj = json.loads(header)
    except json.JSONDecodeError as error:
        raise SafetensorsError(f"parsing safetensors header JSON: {error}") from error
    if not isinstance(obj, dict):
        raise SafetensorsError("expected safetensors header object")
    entries, spans = {}, []
    for name, value in obj.items():
        if name == "__metadata__":
            if not isinstance(value, dict) or not all(isinstance(v, str) for v in value.values()):
                raise SafetensorsError("non-string safetensors metadata")
            continue
        if not isinstance(value, dict) or not isinstance(value.get("dtype"), str):
            raise SafetensorsError(f"missing tensor dtype for {name}")
        if value["dtype"] not in _DTYPES:
            raise SafetensorsError(f"unsupported safetensors dtype {value['dtype']} for {name}")
        dtype, size = _DTYPES[value["dtype"]]
        shape = value.get("shape")
        if not isinstance(shape, list) or not all(isinstance(d, int) and not isinstance(d, bool) and d >= 0 for d in shape):
            raise SafetensorsError(f"missing tensor shape for {name}")
        count = 1
        for d in shape:
            count *= d
        offsets = value.get("data_offsets")
        if (not isinstance(offsets, list) or len(offsets) != 2
                or not all(isinstance(o, int) and not isinstance(o, bool) and o >= 0 for o in offsets)):
            raise SafetensorsError(f"expected two tensor offsets for {name}")
        start, end = offsets
        if not (start <= end <= data_len and end - start == count * size):
            raise SafetensorsError(f"invalid safetensors extent for {name}")
        entries[name] = TensorEntry(dtype, tuple(shape), start, end - start)
        spans.append((start, end))
    spans.sort()
    cursor = 0
    for start, end in spans:
        if start != cursor:
            raise SafetensorsError("safetensors data has a gap or overlapping tensors")
        cursor = end
    if cursor != data_len:
        raise SafetensorsError("unindexed safetensors data")
    return entries


class Shard:
    """One .safetensors file, memory-mapped."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._file = open(path, "rb")
        except OSError as error:
            raise SafetensorsError(f"opening {path}: {error}") from error
        head = self._file.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: reading safetensors header size")
        (length,) = struct.unpack("<Q", head)
        if not (0 < length <= 100_000_000 and length <= size - 8):
            raise SafetensorsError(f"{path}: invalid safetensors header length")
        header = self._file.read(length)
        try:
            self.entries = parse_header(header, size - 8 - length)
        except SafetensorsError as error:
            raise SafetensorsError(f"validating {path}: {error}") from error
        self.data_offset = 8 + length
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def read(self, name: str) -> torch.Tensor:
        entry = self.entries[name]
        begin = self.data_offset + entry.start
        if entry.nbytes == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        raw = torch.frombuffer(bytearray(self._map[begin:begin + entry.nbytes]), dtype=torch.uint8)
        return raw.view(entry.dtype).reshape(entry.shape)


class Archive:
    """All tensors of a model folder, by name."""

    def __init__(self, model_dir: str):
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self.where = {}
        self.shards = {}
        if os.path.exists(index_path):
            with open(index_path, "r", encoding="utf-8") as f:
                index = json.load(f)
            weight_map = index.get("weight_map")
            if not isinstance(weight_map, dict):
                raise SafetensorsError(f"{index_path}: missing weight_map")
            for name, shard in weight_map.items():
                if shard not in self.shards:
                    self.shards[shard] = Shard(os.path.join(model_dir, shard))
                if name not in self.shards[shard].entries:
                    raise SafetensorsError(f"{index_path}: {name} is not in shard {shard}")
                self.where[name] = shard
            for shard, opened in self.shards.items():
                for name in opened.entries:
                    if self.where.get(name) != shard:
                        raise SafetensorsError(f"{shard}: tensor {name} is not in the index")
        elif os.path.exists(single):
            self.shards["model.safetensors"] = Shard(single)
            for name in self.shards["model.safetensors"].entries:
                self.where[name] = "model.safetensors"
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")

    def names(self) -> list:
        return sorted(self.where)

    def entry(self, name: str) -> TensorEntry:
        return self.shards[self.where[name]].entries[name]

    def read(self, name: str) -> torch.Tensor:
        if name not in self.where:
            raise SafetensorsError(f"missing tensor {name}")
        return self.shards[self.where[name]].read(name)


def write_safetensors(path: str, tensors: dict) -> None:
    """Write tensors (name -> CPU tensor) as one safetensors file, names in sorted order."""
    header, cursor = {}, 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} for {name}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [cursor, cursor + nbytes]}
        cursor += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
