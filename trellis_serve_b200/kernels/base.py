"""The contract a kernel backend implements, as the reference states it
(cuda/src/sglang_exl3/kernels/base.py:1-80 of 0xSero/trellis-serve): backends see matrix specs, tensors and a
caller-owned workspace; they never allocate, synchronise or tune on the run path after `warm()`; a key a backend
cannot serve is refused with a reason at load time, not with a failure at run time.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Any, Protocol, Sequence, runtime_checkable


class Op(enum.Enum):
    LINEAR = "linear"
    MOE = "moe"


class ParityClass(enum.Enum):
    BIT_EXACT = "bit_exact"      # decoded weights identical to the reference decoder
    NUMERICAL = "numerical"      # same math, different accumulation order


@dataclass(frozen=True)
class KernelKey:
    op: Op
    layout_class: tuple          # ((k, n, 2K, codebook), ...) per logical matrix
    rows_bucket: int
    in_dtype: str
    out_dtype: str
    device_capability: tuple[int, int]


@dataclass(frozen=True)
class Support:
    ok: bool
    reason: str = ""


@dataclass(frozen=True)
class BackendStatus:
    available: bool
    version: str = ""
    missing: tuple[str, ...] = ()
    detail: str = ""


@dataclass(frozen=True)
class WorkspaceSpec:
    nbytes: int
    alignment: int = 256


@runtime_checkable
class Backend(Protocol):
    name: str

    def probe(self) -> BackendStatus: ...
    def supports(self, key: KernelKey) -> Support: ...
    def parity(self, key: KernelKey) -> ParityClass: ...
    def graph_safe(self, key: KernelKey) -> bool: ...
    def workspace(self, key: KernelKey, max_rows: int) -> WorkspaceSpec: ...
    def prepare_linear(self, layout: Any, tensors: Sequence[dict]) -> Any: ...
    def warm(self, handle: Any, key: KernelKey, workspace: Any) -> None: ...
    def run_linear(self, handle: Any, x: Any, out: Any, workspace: Any) -> None: ...
