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
    def prepare_moe(self, gate: Sequence[Any], up: Sequence[Any], down: Sequence[Any], tensors: dict) -> Any: ...
    def warm(self, handle: Any, key: KernelKey, workspace: Any) -> None: ...
    def run_linear(self, handle: Any, x: Any, out: Any, workspace: Any) -> None: ...
    def run_moe(self, handle: Any, x: Any, topk_ids: Any, topk_weights: Any, out: Any, workspace: Any, expert_map: Any) -> None: ...


_CODEBOOK_IDS = {"3inst": 0, "mcg": 1, "mul1": 2}


def _matrix_reason(m: tuple) -> str:
    """Why one (k, n, twice the bitrate, codebook) entry cannot be served; empty if it can."""
    if m[2] % 2 or not 4 <= m[2] <= 16:
        return f"integer bitrates 2..8 only, got {m[2] / 2:g}"
    if m[3] not in _CODEBOOK_IDS:
        return f"unknown codebook {m[3]!r}"
    if m[0] % 128 or m[1] % 128:
        return "stored widths must be multiples of 128"
    return ""


class B200Backend:
    """The contract over libexl3_b200: dense EXL3 modules and routed experts on sm_100.

    Dense: `prepare_linear` takes a `format.FusedLayout` and, per logical matrix, its stored tensors {"trellis", "suh",
    "svh"} on the device; the handle it returns is the tuple `kernels.linear.prepare` gives plus the codebook number and
    the true output widths.  Routed experts: `prepare_moe` takes the experts' specs per projection and
    tensors = {"gate": [...], "up": [...], "down": [...]} (one dict per expert, same keys), optionally "expert_map" (an
    engine's int32 global -> local id map, -1 for experts held elsewhere); the handle is a `kernels.moe.MixedPack`.
    A key for routed experts describes one expert: layout_class = (gate, up, down) entries; its rows are tokens.

    The workspace is one zero-filled uint8 tensor of `workspace(key, max_rows).nbytes`, owned by the caller; the run
    calls carve it up and allocate nothing.  `max_top_k` / `max_experts` bound what a routed-expert workspace is sized for
    (a key does not carry them)."""
    name = "b200"

    def __init__(self, max_top_k: int = 8, max_experts: int = 256):
        self.max_top_k, self.max_experts = max_top_k, max_experts

    def probe(self) -> BackendStatus:
        from . import linear
        return linear.probe()

    def supports(self, key: KernelKey) -> Support:
        if key.device_capability[0] != 10:
            return Support(False, f"built for sm_100, device is sm_{key.device_capability[0]}{key.device_capability[1]}")
        if key.in_dtype not in ("float16", "bfloat16") or key.out_dtype != key.in_dtype:
            return Support(False, "activations and outputs are fp16 or bf16, and of the same type")
        for m in key.layout_class:
            why = _matrix_reason(m)
            if why:
                return Support(False, why)
        if key.op is Op.MOE:
            if len(key.layout_class) != 3:
                return Support(False, "routed experts are described by their gate, up and down matrices")
            gate, up, down = key.layout_class
            if gate[:2] != up[:2] or down[:2] != (gate[1], gate[0]):
                return Support(False, "gate and up share a shape and down mirrors it")
            if len({m[2] for m in key.layout_class}) != 1 or len({m[3] for m in key.layout_class}) != 1:
                return Support(False, "the projections of an expert share bitrate and codebook")
            return Support(True)
        if not 1 <= len(key.layout_class) <= 4:
            return Support(False, "one to four matrices per fused module")
        if len({m[0] for m in key.layout_class}) != 1 or len({m[2] for m in key.layout_class}) != 1 or len({m[3] for m in key.layout_class}) != 1:
            return Support(False, "the matrices of a module share input width, bitrate and codebook")
        return Support(True)

    def parity(self, key: KernelKey) -> ParityClass:
        return ParityClass.NUMERICAL           # decoded weights are bit-exact; sums run in the kernels' own order

    def graph_safe(self, key: KernelKey) -> bool:
        return True

    # ---- workspaces: [decode scratch | many-row scratch] for dense modules, one layer's temporaries for routed experts

    @staticmethod
    def _dense_split(k: int, n_total: int, shards: int, max_rows: int) -> tuple[int, int]:
        from . import linear
        decode = linear.workspace_bytes(min(max_rows, 16), k, n_total, shards)
        many = linear.tc_workspace_bytes(max_rows, k, n_total, shards) if max_rows > 16 else 0
        return (decode + 255) & ~255, many

    def workspace(self, key: KernelKey, max_rows: int) -> WorkspaceSpec:
        if key.op is Op.MOE:
            from . import moe
            hidden, inter = key.layout_class[0][0], key.layout_class[0][1]
            return WorkspaceSpec(moe.layer_workspace_bytes([self.max_experts], hidden, inter, _CODEBOOK_IDS[key.layout_class[0][3]],
                                                           max_rows, self.max_top_k))
        k = key.layout_class[0][0]
        n_total = sum(m[1] for m in key.layout_class)
        return WorkspaceSpec(sum(self._dense_split(k, n_total, len(key.layout_class), max_rows)))

    def prepare_linear(self, layout: Any, tensors: Sequence[dict]) -> Any:
        from . import linear
        packed, suh_cat, svh_cat, ends = linear.prepare([t["trellis"] for t in tensors], [t["suh"] for t in tensors],
                                                        [t["svh"] for t in tensors])
        codebook = _CODEBOOK_IDS[layout.matrices[0].spec.codebook.value]
        return packed, suh_cat, svh_cat, ends, codebook, [m.out_width for m in layout.matrices]

    def prepare_moe(self, gate: Sequence[Any], up: Sequence[Any], down: Sequence[Any], tensors: dict) -> Any:
        from . import moe
        if not (len(gate) == len(up) == len(down) == len(tensors["gate"]) == len(tensors["up"]) == len(tensors["down"])):
            raise ValueError("one spec and one tensor dict per expert and projection")
        books = {s.codebook.value for s in (*gate, *up, *down)}
        if len(books) != 1:
            raise ValueError(f"the experts of a layer share one codebook, got {sorted(books)}")
        cols = lambda proj: tuple([t[name] for t in tensors[proj]] for name in ("trellis", "suh", "svh"))
        pack = moe.prepare_mixed(cols("gate"), cols("up"), cols("down"), _CODEBOOK_IDS[books.pop()])
        pack.engine_maps = {}
        if tensors.get("expert_map") is not None:
            self._composed_maps(pack, tensors["expert_map"])
        return pack

    @staticmethod
    def _composed_maps(pack: Any, expert_map: Any) -> list:
        """Per bitrate class: engine's global id -> the class's local id (through the pack's own id), cached per map."""
        import torch
        key = (expert_map.data_ptr(), expert_map.numel())
        if key not in pack.engine_maps:
            em = expert_map.to(torch.int64)
            held = em >= 0
            out = []
            for cmap in pack.expert_maps:
                m = torch.full_like(em, -1, dtype=torch.int32)
                m[held] = cmap[em[held]]
                out.append(m.contiguous())
            pack.engine_maps[key] = out
        return pack.engine_maps[key]

    def warm(self, handle: Any, key: KernelKey, workspace: Any) -> None:
        """Launches every kernel instance the key can reach once (zero inputs, results discarded), so that every lazy
        piece of set-up is behind us: after this, run_linear / run_moe for the key neither allocate nor synchronise."""
        import torch
        dtype = torch.float16 if key.in_dtype == "float16" else torch.bfloat16
        if key.op is Op.MOE:
            dev = handle.packs[0].w13.device
            top_k = min(self.max_top_k, handle.num_experts)
            for tokens in sorted({1, key.rows_bucket}):
                x = torch.zeros((tokens, handle.hidden), dtype=dtype, device=dev)
                ids = torch.arange(tokens * top_k, device=dev, dtype=torch.int32).reshape(tokens, top_k) % handle.num_experts
                w = torch.full((tokens, top_k), 1.0 / top_k, dtype=torch.float32, device=dev)
                self.run_moe(handle, x, ids, w, torch.empty_like(x), workspace, None)
            torch.cuda.synchronize(dev)
            return
        from . import linear
        packed = handle[0]
        k, n_total = packed.shape[1] * 128, packed.shape[0] * 128
        if workspace is None:                                   # the module's own scratch: make it large enough now
            linear.reserve_workspace(packed.device, self._dense_split(k, n_total, len(handle[3]) + 1, min(key.rows_bucket, 16))[0])
        buckets = {r for r in (1, 2, 3, 8, 9, 16, 17, 128, 256, 257, 384, 512, 1024) if r < key.rows_bucket} | {key.rows_bucket}
        for rows in sorted(buckets):
            x = torch.zeros((rows, k), dtype=dtype, device=packed.device)
            self.run_linear(handle, x, torch.empty((rows, n_total), dtype=dtype, device=packed.device), workspace)
        torch.cuda.synchronize(packed.device)

    def run_linear(self, handle: Any, x: Any, out: Any, workspace: Any) -> None:
        from .. import _lib
        from ..runtime.ops import prefers_decode
        from . import linear
        packed, suh_cat, svh_cat, ends, codebook, _ = handle
        k, n_total = packed.shape[1] * 128, packed.shape[0] * 128
        rows = x.shape[0]
        decode = rows <= 16 or prefers_decode(rows, k, n_total, _lib.sm_count(packed.device.index))
        if workspace is None:
            (linear.run if decode else linear.run_tc)(x, packed, suh_cat, svh_cat, ends, codebook, out=out)
            return
        cut = self._dense_split(k, n_total, len(ends) + 1, 16)[0]
        if decode:
            linear.run(x, packed, suh_cat, svh_cat, ends, codebook, out=out, workspace=workspace[:cut])
        else:
            linear.run_tc(x, packed, suh_cat, svh_cat, ends, codebook, out=out, workspace=workspace[cut:])

    def run_moe(self, handle: Any, x: Any, topk_ids: Any, topk_weights: Any, out: Any, workspace: Any, expert_map: Any) -> None:
        """`expert_map` (engine's global -> local ids, -1 elsewhere): pass the same tensor to prepare_moe so that its
        composition with the pack's own maps is built at load time; a map first seen here is composed (and allocated) once."""
        from . import moe
        maps = None if expert_map is None else self._composed_maps(handle, expert_map)
        if workspace is None:
            import torch
            need = moe.layer_workspace_bytes([p.num_experts for p in handle.packs], handle.hidden, handle.inter, handle.codebook,
                                             x.shape[0], topk_ids.shape[1])
            workspace = moe._reserve(x.device, need)
        moe.run_layer(x, topk_weights, topk_ids, handle, out, workspace, maps)
