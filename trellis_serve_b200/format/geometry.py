"""Cutting a stored EXL3 matrix into tensor-parallel shares without touching its values.

The input and output rotations act on independent blocks of 128 elements and the trellis holds independent 16 x 16
tiles.  A share that starts and ends on a multiple of 128 therefore consists of whole rotation blocks and whole tiles:
its trellis slice with the matching piece of the sign vector decodes to exactly the corresponding rows (or columns) of
the full matrix.  Other boundaries cannot be served by slicing and are rejected with the reason, so that a caller can
replicate the matrix instead.  Public names and rules are those of core/src/trellis_core/format/geometry.py of
0xSero/trellis-serve (column shares :55-59, row shares :62-66, KV replication :77-83).
"""
from __future__ import annotations

from dataclasses import dataclass

from .spec import BLOCK, TILE, MatrixSpec

_AXIS_OF = {"input": 0, "output": 1}              # trellis dimension a share of that side is cut along


class SplitError(ValueError):
    """Raised when a share cannot be expressed as a slice of the stored tensors."""


@dataclass(frozen=True)
class Narrow:
    """torch.narrow arguments."""
    dim: int
    start: int
    length: int


@dataclass(frozen=True)
class MatrixSlice:
    """Per stored tensor, the narrow that yields one rank's share (None: the tensor is used whole).  `keep_bias` tells
    whether this share adds the bias at all: row shares produce partial sums, so only one of them may."""
    trellis: Narrow
    suh: Narrow | None
    svh: Narrow | None
    bias: Narrow | None
    keep_bias: bool

    def sliced_dims(self, spec: MatrixSpec) -> tuple[int, int]:
        rows = spec.k if self.suh is None else self.suh.length
        cols = spec.n if self.svh is None else self.svh.length
        return rows, cols


def ceil_block(width: int) -> int:
    """Smallest multiple of the rotation block that holds `width` elements."""
    blocks, rest = divmod(width, BLOCK)
    return (blocks + (rest > 0)) * BLOCK


def _share(spec: MatrixSpec, side: str, start: int, size: int) -> MatrixSlice:
    width = spec.k if side == "input" else spec.n
    stop = start + size
    inside = 0 <= start < stop <= width
    if not inside:
        raise SplitError(f"{spec.key}: {side} range [{start}, {stop}) is outside the stored width {width}")
    if (start | size) % BLOCK:
        raise SplitError(f"{spec.key}: {side} range [{start}, {stop}) is not aligned to the {BLOCK}-wide Hadamard "
                         f"blocks; this matrix cannot be sliced there (replicate it instead)")
    tiles = Narrow(_AXIS_OF[side], start // TILE, size // TILE)
    elems = Narrow(0, start, size)
    if side == "output":                          # whole input: every share sees all of suh, its own svh and bias
        return MatrixSlice(tiles, suh=None, svh=elems, bias=elems, keep_bias=True)
    return MatrixSlice(tiles, suh=elems, svh=None, bias=None, keep_bias=(start == 0))


def column_slice(spec: MatrixSpec, start: int, size: int) -> MatrixSlice:
    """Share of the output columns [start, start + size): q / k / v, gate / up, lm_head."""
    return _share(spec, "output", start, size)


def row_slice(spec: MatrixSpec, start: int, size: int) -> MatrixSlice:
    """Share of the input rows [start, start + size): o_proj, down_proj.  The shares' outputs are partial sums."""
    return _share(spec, "input", start, size)


def even_shard(width: int, tp_size: int, tp_rank: int) -> tuple[int, int]:
    """(start, size) of rank `tp_rank` when `width` is divided evenly."""
    size, rest = divmod(width, tp_size)
    if rest:
        raise SplitError(f"width {width} is not divisible by tp_size {tp_size}")
    return size * tp_rank, size


def kv_shard_index(tp_size: int, tp_rank: int, num_kv_heads: int) -> tuple[int, int]:
    """(which share, of how many) a rank takes of a k / v projection.  With more ranks than KV heads every head is held
    by tp_size / num_kv_heads consecutive ranks."""
    if num_kv_heads >= tp_size:
        return tp_rank, tp_size
    copies, rest = divmod(tp_size, num_kv_heads)
    if rest:
        raise SplitError(f"tp_size {tp_size} is not a multiple of num_kv_heads {num_kv_heads}")
    return tp_rank // copies, num_kv_heads


def admissible_tp_degrees(width: int, candidates=(1, 2, 4, 8, 16)) -> list[int]:
    """The degrees among `candidates` whose even shares of `width` are block-aligned (1 always is)."""
    ok = []
    for tp in candidates:
        size, rest = divmod(width, tp)
        if rest == 0 and (tp == 1 or size % BLOCK == 0):
            ok.append(tp)
    return ok
