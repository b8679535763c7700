"""Fused run-time modules seen from the format side.

An engine merges some projections into one module (q|k|v, gate|up): several stored EXL3 matrices read the same input and
write neighbouring column spans of one output.  The matrices stay independent (own sign vectors, possibly own bitrate and
codebook), so the description is just the ordered list with each matrix's true output width; how the group is launched
is up to the backend.  Names follow core/src/trellis_core/format/layout.py of 0xSero/trellis-serve.
"""
from __future__ import annotations

import enum
import itertools
from dataclasses import dataclass
from typing import Hashable, Sequence

from .spec import MatrixSpec


class FusionKind(enum.Enum):
    SINGLE = "single"              # one matrix
    UNIFORM = "uniform"            # same shape, bitrate and codebook throughout, nothing padded
    SHARD_MAP = "shard_map"        # anything else that shares the input
    SEQUENTIAL = "sequential"      # fallback a backend may choose: one launch per matrix


@dataclass(frozen=True)
class LogicalMatrix:
    shard_id: Hashable             # the engine's name for this part of the module ("q", 0, None ...)
    spec: MatrixSpec
    out_width: int                 # true output columns (the stored width is padded to 128)


@dataclass(frozen=True)
class FusedLayout:
    matrices: tuple[LogicalMatrix, ...]

    def __post_init__(self):
        if len(self.matrices) == 0:
            raise ValueError("a fused layout needs at least one matrix")
        widths_in = {m.spec.k for m in self.matrices}
        if len(widths_in) > 1:
            raise ValueError(f"fused matrices must share their input width, got {sorted(widths_in)}")
        bad = next((m for m in self.matrices if m.out_width < 1 or m.out_width > m.spec.n), None)
        if bad is not None:
            raise ValueError(f"{bad.spec.key}: out_width {bad.out_width} does not fit stored width {bad.spec.n}")

    @property
    def in_width(self) -> int:
        return self.matrices[0].spec.k

    @property
    def out_width(self) -> int:
        return sum(m.out_width for m in self.matrices)

    def spans(self) -> list[tuple[int, int]]:
        """(first column, width) of every matrix in the module's output."""
        widths = [m.out_width for m in self.matrices]
        starts = itertools.accumulate([0] + widths[:-1])
        return list(zip(starts, widths))

    @property
    def best_fusion(self) -> FusionKind:
        first, rest = self.matrices[0], self.matrices[1:]
        if not rest:
            return FusionKind.SINGLE
        alike = all(m.spec.same_kernel_class(first.spec) for m in rest)
        unpadded = all(m.out_width == m.spec.n for m in self.matrices)
        return FusionKind.UNIFORM if alike and unpadded else FusionKind.SHARD_MAP


def make_layout(shard_ids: Sequence[Hashable], specs: Sequence[MatrixSpec], out_widths: Sequence[int]) -> FusedLayout:
    if len({len(shard_ids), len(specs), len(out_widths)}) != 1:
        raise ValueError("shard_ids, specs and out_widths must have the same length")
    parts = (LogicalMatrix(sid, spec, width) for sid, spec, width in zip(shard_ids, specs, out_widths))
    return FusedLayout(tuple(parts))
