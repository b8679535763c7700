"""What a kernel backend promises, and the B200 backend as an object that keeps those promises.

The reference states the contract in cuda/src/sglang_exl3/kernels/base.py:1-80 (0xSero/trellis-serve); the type and
method names below are its names, so code written against that contract can hold this backend.  In short:

  * a backend is handed matrix descriptions, tensors and scratch memory owned by the caller;
  * whatever it cannot serve it says at load time (`supports` gives the reason), never by failing at run time;
  * after `warm()` its run path neither allocates, nor synchronises, nor tunes, so it can be captured in a CUDA graph.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Any, Protocol, Sequence, runtime_checkable


class Op(enum.Enum):
    LINEAR = "linear"
    MOE = "moe"


class ParityClass(enum.Enum):
    """How close to the reference decoder a backend's results are for a key."""
    BIT_EXACT = "bit_exact"        # the decoded weights are the reference decoder's, bit for bit
    NUMERICAL = "numerical"        # same arithmetic, other order of accumulation


@dataclass(frozen=True)
class KernelKey:
    """Everything a kernel choice may depend on."""
    op: Op
    layout_class: tuple            # one (k, n, twice the bitrate, codebook name) per logical matrix of the module
    rows_bucket: int               # upper bound of the rows per call this key is for
    in_dtype: str
    out_dtype: str
    device_capability: tuple[int, int]


@dataclass(frozen=True)
class Support:
    ok: bool
    reason: str = ""               # why not, in words a user can act on


@dataclass(frozen=True)
class BackendStatus:
    """Outcome of `probe()`: is the backend usable in this process at all."""
    available: bool
    version: str = ""
    missing: tuple[str, ...] = ()
    detail: str = ""


@dataclass(frozen=True)
class WorkspaceSpec:
    """Scratch the caller has to provide (zero-filled once)."""
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


_CODEBOOK_IDS = {"3inst": 0, "mcg": 1, "mul1": 2}


class B200Backend:
    """The contract over libexl3_b200: dense EXL3 modules on sm_100.  `prepare_linear` takes a `format.FusedLayout` and,
    per logical matrix, its stored tensors {"trellis", "suh", "svh"} on the device; the handle it returns is the tuple
    `kernels.linear.prepare` gives plus the codebook number and the true output widths."""
    name = "b200"

    def probe(self) -> BackendStatus:
        from . import linear
        return linear.probe()

    def supports(self, key: KernelKey) -> Support:
        if key.op is not Op.LINEAR:
            return Support(False, "this object serves dense modules; routed experts go through kernels.moe")
        if key.device_capability[0] != 10:
            return Support(False, f"built for sm_100, device is sm_{key.device_capability[0]}{key.device_capability[1]}")
        if key.in_dtype not in ("float16", "bfloat16") or key.out_dtype != key.in_dtype:
            return Support(False, "activations and outputs are fp16 or bf16, and of the same type")
        if not 1 <= len(key.layout_class) <= 4:
            return Support(False, "one to four matrices per fused module")
        ks = {m[0] for m in key.layout_class}
        rates = {m[2] for m in key.layout_class}
        books = {m[3] for m in key.layout_class}
        if len(ks) != 1 or len(rates) != 1 or len(books) != 1:
            return Support(False, "the matrices of a module share input width, bitrate and codebook")
        twice = next(iter(rates))
        if twice % 2 or not 4 <= twice <= 16:
            return Support(False, f"integer bitrates 2..8 only, got {twice / 2:g}")
        if next(iter(books)) not in _CODEBOOK_IDS:
            return Support(False, f"unknown codebook {next(iter(books))!r}")
        if any(m[0] % 128 or m[1] % 128 for m in key.layout_class):
            return Support(False, "stored widths must be multiples of 128")
        return Support(True)

    def parity(self, key: KernelKey) -> ParityClass:
        return ParityClass.NUMERICAL           # decoded weights are bit-exact; sums run in the kernels' own order

    def graph_safe(self, key: KernelKey) -> bool:
        return True

    def workspace(self, key: KernelKey, max_rows: int) -> WorkspaceSpec:
        from . import linear
        k = key.layout_class[0][0]
        n_total = sum(m[1] for m in key.layout_class)
        return WorkspaceSpec(linear.workspace_bytes(max_rows, k, n_total, len(key.layout_class)))

    def prepare_linear(self, layout: Any, tensors: Sequence[dict]) -> Any:
        from . import linear
        packed, suh_cat, svh_cat, ends = linear.prepare([t["trellis"] for t in tensors], [t["suh"] for t in tensors],
                                                        [t["svh"] for t in tensors])
        codebook = _CODEBOOK_IDS[layout.matrices[0].spec.codebook.value]
        return packed, suh_cat, svh_cat, ends, codebook, [m.out_width for m in layout.matrices]

    def warm(self, handle: Any, key: KernelKey, workspace: Any) -> None:
        from . import linear
        packed = handle[0]
        spec = self.workspace(key, key.rows_bucket)
        linear.reserve_workspace(packed.device, spec.nbytes)       # the last allocation before the run path

    def run_linear(self, handle: Any, x: Any, out: Any, workspace: Any) -> None:
        from . import linear
        packed, suh_cat, svh_cat, ends, codebook, _ = handle
        linear.run(x, packed, suh_cat, svh_cat, ends, codebook, out=out)
