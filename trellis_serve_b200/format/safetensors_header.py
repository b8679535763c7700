"""What a safetensors shard contains, learned from its header alone.

A shard is an unsigned 64-bit little-endian length, that many bytes of JSON, then the tensor data.  The JSON maps every
tensor name to its dtype string, shape and [begin, end) byte range inside the data section; the optional
`__metadata__` entry holds free-form strings.  Nothing here reads tensor data.  Function names and error behaviour follow
core/src/trellis_core/format/safetensors_header.py of 0xSero/trellis-serve.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass

from .spec import FormatError, TensorInfo

_LENGTH = struct.Struct("<Q")
_HEADER_LIMIT = 2 ** 30                     # a larger header means this is not a safetensors file


@dataclass(frozen=True)
class ShardHeader:
    file: str                                # file name the tensors will be reported under
    metadata: dict
    tensors: dict                            # name -> TensorInfo


def _tensor_info(name: str, entry: dict, file: str) -> TensorInfo:
    begin, end = entry["data_offsets"]
    if end < begin:
        raise FormatError(f"{file}: {name}: data_offsets [{begin}, {end}) is reversed")
    return TensorInfo(name=name, dtype=entry["dtype"], shape=tuple(entry["shape"]), file=file, nbytes=end - begin)


def parse_header(raw: bytes, file: str = "") -> ShardHeader:
    """`raw` = the JSON bytes of a shard's header."""
    try:
        entries = json.loads(raw)
    except ValueError as err:
        raise FormatError(f"{file}: safetensors header is not valid JSON: {err}") from None
    metadata = entries.get("__metadata__") or {}
    tensors = {name: _tensor_info(name, entry, file) for name, entry in entries.items() if name != "__metadata__"}
    return ShardHeader(file=file, metadata=metadata, tensors=tensors)


def read_header(path) -> ShardHeader:
    """Header of the shard at `path`; tensors are reported under the file's base name."""
    path = os.fspath(path)
    with open(path, "rb") as shard:
        prefix = shard.read(_LENGTH.size)
        if len(prefix) < _LENGTH.size:
            raise FormatError(f"{path}: too short to be a safetensors file")
        (size,) = _LENGTH.unpack(prefix)
        if size < 2 or size > _HEADER_LIMIT:
            raise FormatError(f"{path}: implausible safetensors header length {size}")
        body = shard.read(size)
    if len(body) < size:
        raise FormatError(f"{path}: truncated safetensors header")
    return parse_header(body, os.path.basename(path))
