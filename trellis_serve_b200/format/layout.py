"""Logical matrices of a fused run-time module (q|k|v, gate|up ...): an ordered group of independent EXL3 matrices
that share an input and write adjacent output spans, each with its own suh, K and codebook.  Same description as
core/src/trellis_core/format/layout.py of 0xSero/trellis-serve; how a group is launched is the backend's business.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Hashable, Sequence

from .spec import MatrixSpec


@dataclass(frozen=True)
class LogicalMatrix:
    shard_id: Hashable
    spec: MatrixSpec
    out_width: int


class FusionKind(enum.Enum):
    SINGLE = "single"
    UNIFORM = "uniform"
    SHARD_MAP = "shard_map"
    SEQUENTIAL = "sequential"


@dataclass(frozen=True)
class FusedLayout:
    matrices: tuple[LogicalMatrix, ...]

    def __post_init__(self):
        if not self.matrices:
            raise ValueError("a fused layout needs at least one matrix")
        ks = sorted({m.spec.k for m in self.matrices})
        if len(ks) != 1:
            raise ValueError(f"fused matrices must share their input width, got {ks}")
        for m in self.matrices:
            if not 0 < m.out_width <= m.spec.n:
                raise ValueError(f"{m.spec.key}: out_width {m.out_width} does not fit stored width {m.spec.n}")

    @property
    def in_width(self) -> int:
        return self.matrices[0].spec.k

    @property
    def out_width(self) -> int:
        return sum(m.out_width for m in self.matrices)

    def spans(self) -> list[tuple[int, int]]:
        spans, at = [], 0
        for m in self.matrices:
            spans.append((at, m.out_width))
            at += m.out_width
        return spans

    @property
    def best_fusion(self) -> FusionKind:
        if len(self.matrices) == 1:
            return FusionKind.SINGLE
        head = self.matrices[0].spec
        uniform = all(m.spec.same_kernel_class(head) and m.out_width == m.spec.n for m in self.matrices)
        return FusionKind.UNIFORM if uniform else FusionKind.SHARD_MAP


def make_layout(shard_ids: Sequence[Hashable], specs: Sequence[MatrixSpec], out_widths: Sequence[int]) -> FusedLayout:
    if not len(shard_ids) == len(specs) == len(out_widths):
        raise ValueError("shard_ids, specs and out_widths must have the same length")
    return FusedLayout(tuple(LogicalMatrix(*t) for t in zip(shard_ids, specs, out_widths)))
