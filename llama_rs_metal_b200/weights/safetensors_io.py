"""Reading and writing SafeTensors files without a library.

Layout: 8-byte little-endian header length, a JSON header mapping each tensor
name to {dtype, shape, data_offsets}, then the raw bytes. A folder holds either
`model.safetensors` or `model.safetensors.index.json` (`weight_map`) with
shards; the checks are those of the reference's reader
(crates/model-format/src/mlx/safetensors.rs:19-92).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Tuple

import torch

from ..errors import InvalidError, UnsupportedError

JSON_LIMIT = 128 << 20  # safetensors.rs:21-23

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    """One tensor of an open checkpoint; `load()` gives a CPU tensor over the mapping."""

    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    file: str
    begin: int
    end: int
    _buffer: object = None

    @property
    def nbytes(self) -> int:
        return self.end - self.begin

    def load(self) -> torch.Tensor:
        count = 1
        for s in self.shape:
            count *= s
        if count == 0:
            return torch.empty(self.shape, dtype=self.dtype)
        flat = torch.frombuffer(self._buffer, dtype=self.dtype, count=count, offset=self.begin)
        return flat.view(self.shape)


def _open_file(path: str) -> Dict[str, TensorEntry]:
    size = os.path.getsize(path)
    if size < 8:
        raise InvalidError(f"{path}: truncated SafeTensors file")
    handle = open(path, "rb")
    (header_len,) = struct.unpack("<Q", handle.read(8))
    if header_len > JSON_LIMIT or 8 + header_len > size:
        handle.close()
        raise InvalidError(f"{path}: truncated or oversized SafeTensors header")
    try:
        header = json.loads(handle.read(header_len).decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError):
        handle.close()
        raise InvalidError(f"{path}: SafeTensors header is not valid JSON") from None
    if not isinstance(header, dict):
        handle.close()
        raise InvalidError(f"{path}: SafeTensors header must be an object")
    buffer = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_COPY)
    handle.close()
    base = 8 + header_len
    entries = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype_name, shape, (begin, end) = meta["dtype"], tuple(meta["shape"]), meta["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise InvalidError(f"{path}: malformed entry for {name}") from None
        if dtype_name not in _DTYPES:
            raise UnsupportedError(f"{path}: {name} has unsupported dtype {dtype_name}")
        dtype = _DTYPES[dtype_name]
        count = 1
        for s in shape:
            count *= s
        if end - begin != count * torch.empty((), dtype=dtype).element_size() or base + end > size \
                or begin < 0:
            raise InvalidError(f"{path}: truncated or inconsistent data for {name}")
        entries[name] = TensorEntry(name, dtype, shape, path, base + begin, base + end, buffer)
    return entries


def open_checkpoint(model_dir: str) -> Dict[str, TensorEntry]:
    """Every tensor of a model folder by its stored name (single file or indexed shards)."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        if os.path.getsize(index) > JSON_LIMIT:
            raise InvalidError(f"{index}: index larger than {JSON_LIMIT} bytes")
        try:
            with open(index, "r", encoding="utf-8") as handle:
                weight_map = json.load(handle)["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError):
            raise InvalidError(f"{index}: no weight_map") from None
        if not isinstance(weight_map, dict):
            raise InvalidError(f"{index}: weight_map must be an object")
        shards = sorted(set(weight_map.values()))
        entries: Dict[str, TensorEntry] = {}
        for shard in shards:
            # safetensors.rs:41-47: a plain file name that ends in .safetensors
            if not isinstance(shard, str) or not shard.endswith(".safetensors") \
                    or os.path.basename(shard) != shard or shard.startswith("."):
                raise InvalidError(f"{index}: unsafe shard name {shard!r}")
            found = _open_file(os.path.join(model_dir, shard))
            for name, entry in found.items():
                if weight_map.get(name) != shard:  # safetensors.rs:64-72
                    raise InvalidError(f"{shard}: tensor {name} is not assigned to this shard by the index")
                if name in entries:  # safetensors.rs:79-81
                    raise InvalidError(f"duplicate tensor {name}")
                entries[name] = entry
        absent = sorted(set(weight_map) - set(entries))  # safetensors.rs:84-90
        if absent:
            raise InvalidError(f"{index}: tensors missing from shards: {', '.join(absent)}")
        return entries
    if os.path.isfile(single):
        return _open_file(single)
    raise InvalidError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write CPU tensors to one SafeTensors file, names in sorted order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise UnsupportedError(f"{name}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * ((8 - len(encoded) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for raw in blobs:
            handle.write(raw)
