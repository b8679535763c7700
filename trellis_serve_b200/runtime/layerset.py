"""The EXL3 linears of a stack of transformer layers as one replayable decode step.

A decode step of a dense transformer touches, per layer, four fused EXL3 launches: q|k|v (shared input, three
matrices with their own suh), o, gate|up and down.  `DecodeLayerSet` owns the resident weights of such a stack for
one tensor-parallel rank, pre-binds every launch through the backend functions of `kernels.linear` and captures
the whole step in one CUDA graph, which is how an engine drives the reference's kernels too (warm-up then capture:
cuda/src/sglang_exl3/sglang_glue/moe.py:202-213, cuda/src/sglang_exl3/tools/decode_microbench.py:27-41 of
0xSero/trellis-serve).

Tensor parallelism follows the exact-slicing rules of the format layer (format/geometry.py): q, k, v, gate and up
are split by output columns, o and down by input rows, all at 128-aligned boundaries; the row-parallel outputs
are partial sums that one all-reduce per matrix adds up.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import linear as lin


@dataclass(frozen=True)
class LayerShape:
    hidden: int = 5120
    q_out: int = 5120
    kv_out: int = 1024
    ffn: int = 17408

    def packed_bytes_per_layer(self, K: int) -> int:
        weights = self.hidden * (self.q_out + 2 * self.kv_out) + self.q_out * self.hidden + 3 * self.hidden * self.ffn
        return weights * K // 8


@dataclass
class _Group:
    packed: torch.Tensor
    suh: torch.Tensor
    svh: torch.Tensor
    ends: list
    reduce: bool


def random_packed(k: int, n: int, K: int, gen: torch.Generator, device) -> torch.Tensor:
    """Uniform random resident weights.  The resident layout is a permutation of the stored bits, so uniform bits here
    are uniform bits of the stored trellis (recover it with kernels.linear.unprepare_matrix)."""
    t = torch.randint(-2 ** 31, 2 ** 31 - 1, (n // 128, k // 128, 8, 2, K, 32), dtype=torch.int32, device=device, generator=gen)
    return t


def random_signs(n: int, gen: torch.Generator, device, shards: int = 1) -> torch.Tensor:
    s = torch.randint(0, 2, (shards, n), device=device, generator=gen, dtype=torch.int32) * 2 - 1
    return s.to(torch.float16)


class DecodeLayerSet:
    """`layers` x (qkv, o, gate_up, down) EXL3 groups of one tensor-parallel rank, random-initialised."""

    def __init__(self, layers: int, K: int, codebook: int, rows: int, shape: LayerShape = LayerShape(), tp_rank: int = 0,
                 tp_size: int = 1, seed: int = 100, device: str | torch.device = "cuda:0", group=None,
                 allreduce=None, dtype: torch.dtype = torch.float16, fused_exchange: bool = False):
        self.layers, self.K, self.codebook, self.rows = layers, K, codebook, rows
        self.shape, self.tp_rank, self.tp_size = shape, tp_rank, tp_size
        self.device = torch.device(device)
        self.group = group
        self.allreduce = allreduce
        # fused_exchange (needs a PeerAllReduce in `allreduce`): row-parallel linears sum over the ranks inside their kernel
        self.fused_exchange = bool(fused_exchange and allreduce is not None and tp_size > 1)
        self.dtype = dtype
        for width in (shape.q_out, shape.kv_out, shape.ffn, shape.hidden):
            if width % tp_size or (width // tp_size) % 128:
                raise ValueError(f"width {width} cannot be split over {tp_size} ranks at 128-aligned boundaries")
        h, tp = shape.hidden, tp_size
        q, kv, f = shape.q_out // tp, shape.kv_out // tp, shape.ffn // tp
        gen = torch.Generator(device=self.device)
        self.groups: list[list[_Group]] = []
        for layer in range(layers):
            gen.manual_seed(seed + layer * 1000 + tp_rank)
            qkv = _Group(torch.cat([random_packed(h, w, K, gen, self.device) for w in (q, kv, kv)]),
                         random_signs(h, gen, self.device, 3), random_signs(q + 2 * kv, gen, self.device).view(-1), [q, q + kv], False)
            o = _Group(random_packed(shape.q_out // tp, h, K, gen, self.device), random_signs(shape.q_out // tp, gen, self.device),
                       random_signs(h, gen, self.device).view(-1), [], tp > 1)
            gu = _Group(torch.cat([random_packed(h, f, K, gen, self.device) for _ in range(2)]),
                        random_signs(h, gen, self.device, 2), random_signs(2 * f, gen, self.device).view(-1), [f], False)
            down = _Group(random_packed(f, h, K, gen, self.device), random_signs(f, gen, self.device),
                          random_signs(h, gen, self.device).view(-1), [], tp > 1)
            self.groups.append([qkv, o, gu, down])
        ws = max(lin.workspace_bytes(rows, k, n, s) for k, n, s in
                 ((h, q + 2 * kv, 3), (shape.q_out // tp, h, 1), (h, 2 * f, 2), (f, h, 1)))
        lin.reserve_workspace(self.device, ws)
        # static activations: every linear reads a fixed buffer, as in a captured decode step
        self.x_hidden = torch.zeros((rows, h), dtype=dtype, device=self.device)
        self.x_attn = torch.zeros((rows, shape.q_out // tp), dtype=dtype, device=self.device)
        self.x_ffn = torch.zeros((rows, f), dtype=dtype, device=self.device)
        self.y_qkv = torch.empty((rows, q + 2 * kv), dtype=dtype, device=self.device)
        self.y_o = torch.empty((rows, h), dtype=dtype, device=self.device)
        self.y_gu = torch.empty((rows, 2 * f), dtype=dtype, device=self.device)
        self.y_down = torch.empty((rows, h), dtype=dtype, device=self.device)
        self.graph: torch.cuda.CUDAGraph | None = None
        # up to two rows the GEMV rotates its own input: one launch per group; otherwise rotation + GEMV
        self.launches_per_step = layers * 4 * (1 if rows <= 2 else 2)
        if tp_size > 1 and allreduce is not None and not self.fused_exchange:
            self.launches_per_step += layers * 2             # the stand-alone exchange kernel after o and down

    @property
    def packed_bytes(self) -> int:
        """Packed-weight bytes this rank streams per step."""
        return sum(g.packed.numel() * 4 for layer in self.groups for g in layer)

    def _reduce(self, t: torch.Tensor) -> None:
        if self.tp_size == 1:
            return
        if self.allreduce is not None:
            self.allreduce(t)
        else:
            torch.distributed.all_reduce(t, group=self.group)

    def step(self) -> torch.Tensor:
        """All linears of the stack once, in layer order, on the current stream."""
        for qkv, o, gu, down in self.groups:
            lin.run(self.x_hidden, qkv.packed, qkv.suh, qkv.svh, qkv.ends, self.codebook, out=self.y_qkv)
            if self.fused_exchange:
                lin.run(self.x_attn, o.packed, o.suh, o.svh, o.ends, self.codebook, out=self.y_o, exchange=self.allreduce)
            else:
                lin.run(self.x_attn, o.packed, o.suh, o.svh, o.ends, self.codebook, out=self.y_o)
                self._reduce(self.y_o)
            lin.run(self.x_hidden, gu.packed, gu.suh, gu.svh, gu.ends, self.codebook, out=self.y_gu)
            if self.fused_exchange:
                lin.run(self.x_ffn, down.packed, down.suh, down.svh, down.ends, self.codebook, out=self.y_down, exchange=self.allreduce)
            else:
                lin.run(self.x_ffn, down.packed, down.suh, down.svh, down.ends, self.codebook, out=self.y_down)
                self._reduce(self.y_down)
        return self.y_down

    def capture(self, warmup: int = 2) -> None:
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step()

    def replay(self) -> torch.Tensor:
        if self.graph is None:
            self.capture()
        self.graph.replay()
        return self.y_down

    def forward_host(self, x_hidden: torch.Tensor, x_attn: torch.Tensor, x_ffn: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """End-to-end step with host buffers: pinned inputs are copied to the device, the captured step runs, the last
        layer's output is copied back into `out` (pinned) and the stream is synchronised."""
        self.x_hidden.copy_(x_hidden, non_blocking=True)
        self.x_attn.copy_(x_attn, non_blocking=True)
        self.x_ffn.copy_(x_ffn, non_blocking=True)
        y = self.replay()
        out.copy_(y, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out
