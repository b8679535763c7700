"""Header-only safetensors reader (u64 little-endian header length, JSON header, raw data): names, dtypes, shapes
and byte ranges without touching tensor data.  API of core/src/trellis_core/format/safetensors_header.py."""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass

from .spec import FormatError, TensorInfo

_MAX_HEADER = 1 << 30


@dataclass(frozen=True)
class ShardHeader:
    file: str
    metadata: dict
    tensors: dict


def parse_header(raw: bytes, file: str = "") -> ShardHeader:
    try:
        doc = json.loads(raw)
    except ValueError as e:
        raise FormatError(f"{file}: safetensors header is not valid JSON: {e}") from None
    meta = doc.pop("__metadata__", None) or {}
    tensors = {}
    for name, entry in doc.items():
        lo, hi = entry["data_offsets"]
        if hi < lo:
            raise FormatError(f"{file}: {name}: data_offsets [{lo}, {hi}) is reversed")
        tensors[name] = TensorInfo(name, entry["dtype"], tuple(entry["shape"]), file, hi - lo)
    return ShardHeader(file, meta, tensors)


def read_header(path) -> ShardHeader:
    path = os.fspath(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise FormatError(f"{path}: too short to be a safetensors file")
        (length,) = struct.unpack("<Q", head)
        if not 2 <= length <= _MAX_HEADER:
            raise FormatError(f"{path}: implausible safetensors header length {length}")
        raw = f.read(length)
    if len(raw) != length:
        raise FormatError(f"{path}: truncated safetensors header")
    return parse_header(raw, os.path.basename(path))
