"""Padding and tensor-parallel slicing of stored EXL3 matrices.

Both Hadamard rotations are block-diagonal with 128-wide blocks and the trellis is tiled 16 x 16, so a 128-aligned
slice of (trellis, scale vector) is itself a complete EXL3 matrix that reproduces exactly those rows or columns:
slicing needs no re-quantisation.  Boundaries that are not 128-aligned are refused with a reason.  Same rules and
names as core/src/trellis_core/format/geometry.py of 0xSero/trellis-serve (column_slice :55-59, row_slice :62-66).
"""
from __future__ import annotations

from dataclasses import dataclass

from .spec import BLOCK, TILE, MatrixSpec


def ceil_block(width: int) -> int:
    return (width + BLOCK - 1) // BLOCK * BLOCK


class SplitError(ValueError):
    """The requested shard boundary cannot be produced by slicing."""


@dataclass(frozen=True)
class Narrow:
    dim: int
    start: int
    length: int


@dataclass(frozen=True)
class MatrixSlice:
    """How one rank's share is cut out of the stored tensors; None keeps a tensor whole."""
    trellis: Narrow
    suh: Narrow | None
    svh: Narrow | None
    bias: Narrow | None
    keep_bias: bool

    def sliced_dims(self, spec: MatrixSpec) -> tuple[int, int]:
        return (self.suh.length if self.suh else spec.k), (self.svh.length if self.svh else spec.n)


def _validate(spec: MatrixSpec, side: str, width: int, start: int, size: int) -> None:
    if size <= 0 or start < 0 or start + size > width:
        raise SplitError(f"{spec.key}: {side} range [{start}, {start + size}) is outside the stored width {width}")
    if start % BLOCK or size % BLOCK:
        raise SplitError(f"{spec.key}: {side} range [{start}, {start + size}) is not aligned to the {BLOCK}-wide "
                         f"Hadamard blocks; this matrix cannot be sliced there (replicate it instead)")


def column_slice(spec: MatrixSpec, start: int, size: int) -> MatrixSlice:
    """Output-dimension split (q/k/v, gate/up, lm_head): trellis dim 1, svh and bias are cut, suh stays whole."""
    _validate(spec, "output", spec.n, start, size)
    cols = Narrow(0, start, size)
    return MatrixSlice(Narrow(1, start // TILE, size // TILE), None, cols, cols, True)


def row_slice(spec: MatrixSpec, start: int, size: int) -> MatrixSlice:
    """Input-dimension split (o_proj, down_proj): trellis dim 0 and suh are cut, svh stays whole, the bias is
    added once, by the shard that starts at row 0."""
    _validate(spec, "input", spec.k, start, size)
    return MatrixSlice(Narrow(0, start // TILE, size // TILE), Narrow(0, start, size), None, None, start == 0)


def even_shard(width: int, tp_size: int, tp_rank: int) -> tuple[int, int]:
    if width % tp_size:
        raise SplitError(f"width {width} is not divisible by tp_size {tp_size}")
    size = width // tp_size
    return tp_rank * size, size


def kv_shard_index(tp_size: int, tp_rank: int, num_kv_heads: int) -> tuple[int, int]:
    """(shard index, shard count) of a k/v projection; KV heads are replicated when there are more ranks than heads."""
    if tp_size <= num_kv_heads:
        return tp_rank, tp_size
    if tp_size % num_kv_heads:
        raise SplitError(f"tp_size {tp_size} is not a multiple of num_kv_heads {num_kv_heads}")
    return tp_rank // (tp_size // num_kv_heads), num_kv_heads


def admissible_tp_degrees(width: int, candidates=(1, 2, 4, 8, 16)) -> list[int]:
    return [tp for tp in candidates if width % tp == 0 and (tp == 1 or (width // tp) % BLOCK == 0)]
