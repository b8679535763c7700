"""One decoded token through a dense transformer of EXL3 linears: the step either side of the kernels.

    per layer:  a = RMSNorm(residual)                          -> inside the input rotation of q|k|v       (normed linear)
                q|k|v = EXL3(a);  RoPE(q, k);  KV cache append;  attention over the cache
                o = EXL3(attention)                             -> rotation launch, then the GEMV
                residual += o                                   -> in the epilogue of o (with the stream's sums of squares)
                a = RMSNorm(residual)                           -> inside the input rotation of gate|up
                g|u = EXL3(a);  act = SiLU(g) * u               -> computed inside down's own input rotation (glu linear; from three
                h = EXL3(act);  residual += h                      rows up: silu_mul_rotate ahead of the GEMV); the sum in down's epilogue

Every linear is ONE decode-GEMV launch whose activations were rotated by the kernel ahead of it; rotary embedding, cache
append and attention are stock torch (`scaled_dot_product_attention`): they are not part of the quantized-linear path and
their bytes (the KV read) are reported separately.  `attention="library"` (default) runs the library's own kernel for that part (RoPE + cache append + split-KV attention, merged
by the last CTA to arrive); `attention="torch"` keeps the stock torch ops.  The whole step is captured in one CUDA graph, as an engine captures
it (cuda/src/sglang_exl3/sglang_glue/moe.py:202-213 warms for that purpose; cuda/src/sglang_exl3/tools/decode_microbench.py
:27-41 times launches the same way).

Tensor parallelism: query and KV heads are split over the ranks (with more ranks than KV heads every head is held by
several ranks: format/geometry.py `kv_shard_index`), q|k|v and gate|up by columns, o and down by rows with the exchange
fused into their GEMV (or NCCL).  Weights are random (uniform trellis bits, +-1 sign vectors scaled so that activations
stay in range); the step exists to be timed and to be checked against a float64 restatement, not to produce language.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..format import kv_shard_index
from ..kernels import linear as lin
from .layerset import random_packed, random_signs


@dataclass(frozen=True)
class ModelShape:
    hidden: int = 5120
    q_heads: int = 40
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 17408
    layers: int = 64
    rope_theta: float = 1.0e6
    eps: float = 1.0e-6

    @property
    def q_out(self) -> int:
        return self.q_heads * self.head_dim

    @property
    def kv_out(self) -> int:
        return self.kv_heads * self.head_dim

    def packed_bytes_per_layer(self, K: int) -> int:
        weights = self.hidden * (self.q_out + 2 * self.kv_out) + self.q_out * self.hidden + 3 * self.hidden * self.ffn
        return weights * K // 8

    def kv_bytes_per_token(self, context: int, dtype_bytes: int = 2) -> int:
        """Bytes of keys and values one decoded token reads (all layers, all KV heads)."""
        return self.layers * 2 * self.kv_heads * self.head_dim * context * dtype_bytes


@dataclass
class _Lin:
    packed: torch.Tensor
    suh: torch.Tensor
    svh: torch.Tensor
    ends: list


class DecodeStep:
    """Random-initialised dense transformer of `shape` at `K` bits, one tensor-parallel rank of `tp_size`."""

    def __init__(self, shape: ModelShape, K: int, codebook: int, context: int, rows: int = 1, tp_rank: int = 0, tp_size: int = 1,
                 device="cuda:0", dtype: torch.dtype = torch.float16, seed: int = 400, exchange=None, group=None,
                 attention: str = "library"):
        self.shape, self.K, self.codebook, self.context, self.rows = shape, K, codebook, context, rows
        self.tp_rank, self.tp_size, self.exchange, self.group = tp_rank, tp_size, exchange, group
        self.device, self.dtype, self.attention = torch.device(device), dtype, attention
        s, dev, tp = shape, self.device, tp_size
        if s.q_heads % tp or s.ffn % tp or (s.ffn // tp) % 128 or (s.q_out // tp) % 128:
            raise ValueError(f"{s.q_heads} query heads / ffn {s.ffn} cannot be split over {tp} ranks at 128-aligned boundaries")
        kv_index, kv_parts = kv_shard_index(tp, tp_rank, s.kv_heads)
        self.q_heads, self.kv_heads = s.q_heads // tp, s.kv_heads // kv_parts
        q, kv, f, h = self.q_heads * s.head_dim, self.kv_heads * s.head_dim, s.ffn // tp, s.hidden
        gen = torch.Generator(device=dev)
        scale = lambda n, k: (random_signs(n, gen, dev).view(-1).float() * (1.0 / (1.2437 * math.sqrt(k)))).half()
        self.layers = []
        for layer in range(s.layers):
            gen.manual_seed(seed + layer * 1000 + tp_rank)
            qkv = _Lin(torch.cat([random_packed(h, w, K, gen, dev) for w in (q, kv, kv)]), random_signs(h, gen, dev, 3),
                       scale(q + 2 * kv, h), [q, q + kv])
            o = _Lin(random_packed(q, h, K, gen, dev), random_signs(q, gen, dev, 1), scale(h, s.q_out), [])
            gu = _Lin(torch.cat([random_packed(h, f, K, gen, dev) for _ in range(2)]), random_signs(h, gen, dev, 2), scale(2 * f, h), [f])
            down = _Lin(random_packed(f, h, K, gen, dev), random_signs(f, gen, dev, 1), scale(h, s.ffn), [])
            norms = (1.0 + 0.1 * torch.randn((2, h), device=dev, generator=gen)).to(dtype)
            self.layers.append((qkv, o, gu, down, norms))
        self.final_norm = torch.ones(h, dtype=dtype, device=dev)
        self.workspace = torch.zeros(max(lin.workspace_bytes(rows, k_, n_, sh) for k_, n_, sh in
                                         ((h, q + 2 * kv, 3), (q, h, 1), (h, 2 * f, 2), (f, h, 1))), dtype=torch.uint8, device=dev)
        # KV cache [layer][2][rows, kv heads, context + 1, head_dim]: `context` past positions (random) and one new slot
        self.kv = (torch.randn((s.layers, 2, rows, self.kv_heads, context + 1, s.head_dim), device=dev, generator=gen) * 0.5).to(dtype)
        pos = torch.tensor([float(context)], device=dev)
        inv = 1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, device=dev).float() / s.head_dim))
        ang = pos[:, None] * inv[None, :]
        self.cos, self.sin = torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)          # [1, head_dim / 2]
        # the library's attention kernels: tables by position (the values of the torch path, as fp32), position on the device
        self.cos_table = torch.zeros((context + 1, s.head_dim // 2), dtype=torch.float32, device=dev)
        self.sin_table = torch.zeros_like(self.cos_table)
        self.cos_table[context], self.sin_table[context] = self.cos[0].float(), self.sin[0].float()
        self.position = torch.tensor([context], dtype=torch.int32, device=dev)
        from .. import _lib
        self.att_scratch = torch.zeros(int(_lib.load().exl3_attention_scratch_bytes(rows, self.q_heads, self.kv_heads, context + 1)),
                                       dtype=torch.uint8, device=dev)
        # activations of the chain (static: the captured graph sees fixed addresses)
        mk = lambda w: torch.empty((rows, w), dtype=dtype, device=dev)
        self.h_in = torch.zeros((rows, h), dtype=dtype, device=dev)          # the step's input: the token's embedding
        self.h, self.residual, self.residual2 = mk(h), mk(h), mk(h)        # the residual stream alternates between two buffers
        self.ssq = torch.zeros((rows, h // 128), dtype=torch.float32, device=dev)     # its sums of squares per 128 columns
        self.ssq2 = torch.zeros_like(self.ssq)
        self.qkv, self.attn, self.o_out, self.gu, self.out = mk(q + 2 * kv), mk(q), mk(h), mk(2 * f), mk(h)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.linear_launches = s.layers * 4
        small = 0 if rows <= 2 else 5                                 # normalisation x2, activation and stream x2 kernels: only from three rows up
        self.fused_launches = 1 + s.layers * ((0 if attention == "library" else 1) + small)   # the stream's start (+ rotation ahead of o with stock attention)
        self.attention_launches = s.layers if attention == "library" else None   # RoPE, append, attention and merge in one

    # ---- bytes
    @property
    def packed_bytes(self) -> int:
        return sum(l.packed.numel() * 4 for layer in self.layers for l in layer[:4])

    @property
    def kv_bytes(self) -> int:
        """Key and value bytes this rank reads per step."""
        return self.shape.layers * 2 * self.rows * self.kv_heads * self.context * self.shape.head_dim * self.kv.element_size()

    # ---- the step
    def _rope(self, t: torch.Tensor, heads: int) -> torch.Tensor:
        x = t.view(self.rows, heads, self.shape.head_dim)
        x1, x2 = x[..., : self.shape.head_dim // 2], x[..., self.shape.head_dim // 2:]
        return torch.cat([x1 * self.cos - x2 * self.sin, x2 * self.cos + x1 * self.sin], dim=-1)

    def _attention(self, layer: int, suh_next: torch.Tensor | None = None) -> bool:
        """RoPE, cache append and attention of one layer into `self.attn`.  True when the rotated input of the o projection
        was written as well (the library's merge kernel does that when handed the projection's sign vector)."""
        s, q, kv = self.shape, self.q_heads * self.shape.head_dim, self.kv_heads * self.shape.head_dim
        if self.attention == "library":
            from .. import _lib
            lib, p, st = _lib.load(), lin._ptr, lin._stream(self.device)
            cache, code = self.kv[layer], lin._dtype_code(self.qkv)
            with torch.cuda.device(self.device):
                _lib.check(lib.exl3_rope_decode_attention(p(self.qkv), code, self.rows, self.q_heads, self.kv_heads, s.head_dim,
                                                          p(self.cos_table), p(self.sin_table), p(cache[0]), p(cache[1]), self.context + 1,
                                                          p(self.position), 1.0 / math.sqrt(s.head_dim), p(self.att_scratch),
                                                          self.att_scratch.numel(), p(self.attn), p(suh_next), self.codebook,
                                                          p(self.workspace), self.workspace.numel(), st), "exl3_rope_decode_attention")
            return suh_next is not None
        qh = self._rope(self.qkv[:, :q], self.q_heads).unsqueeze(2)                        # [rows, q heads, 1, d]
        kh = self._rope(self.qkv[:, q:q + kv], self.kv_heads)
        vh = self.qkv[:, q + kv:].view(self.rows, self.kv_heads, s.head_dim)
        cache = self.kv[layer]
        cache[0][:, :, self.context] = kh
        cache[1][:, :, self.context] = vh
        y = torch.nn.functional.scaled_dot_product_attention(qh, cache[0], cache[1], enable_gqa=self.q_heads != self.kv_heads)
        self.attn.copy_(y.reshape(self.rows, q))
        return False

    def _reduce(self, t: torch.Tensor) -> None:
        if self.tp_size > 1 and self.exchange is None:
            torch.distributed.all_reduce(t, group=self.group)

    def step(self) -> torch.Tensor:
        """One token through all layers on the current stream; returns the final normalised hidden state."""
        cb, ws, ex, rows = self.codebook, self.workspace, self.exchange, self.rows
        fused = ex is not None or self.tp_size == 1      # the linears' epilogues carry the residual stream (NCCL sums outside them)
        z, z2, ssq, ssq2 = self.residual, self.residual2, self.ssq, self.ssq2
        lin.residual_ssq(self.h_in, None, z, ssq)           # the stream starts as the token's embedding
        for i, (qkv, o, gu, down, norms) in enumerate(self.layers):
            lin.run_normed(z, ssq, norms[0], self.shape.eps, qkv.packed, qkv.suh, qkv.svh, qkv.ends, cb, self.qkv, ws)
            if not self._attention(i, o.suh):
                lin.rotate_fragments(self.attn, o.suh, cb, ws)
            if fused:
                lin.run_prerotated(rows, o.packed, o.svh, o.ends, cb, self.o_out, ws, exchange=ex, residual=(z, z2, ssq2))
            else:
                lin.run_prerotated(rows, o.packed, o.svh, o.ends, cb, self.o_out, ws)
                self._reduce(self.o_out)
                lin.residual_ssq(self.o_out, z, z2, ssq2)
            lin.run_normed(z2, ssq2, norms[1], self.shape.eps, gu.packed, gu.suh, gu.svh, gu.ends, cb, self.gu, ws)
            if fused:
                lin.run_glu(self.gu, down.packed, down.suh, down.svh, cb, self.h, ws, exchange=ex, residual=(z2, z, ssq))
            else:
                lin.run_glu(self.gu, down.packed, down.suh, down.svh, cb, self.h, ws)
                self._reduce(self.h)
                lin.residual_ssq(self.h, z2, z, ssq)
        self.out.copy_(torch.nn.functional.rms_norm(z.float(), (self.shape.hidden,), self.final_norm.float(), self.shape.eps).to(self.dtype))
        return self.out

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
        return self.out

    def forward_host(self, embedding: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """End to end with host buffers: the token's embedding (pinned) in, the final hidden state (pinned) out."""
        self.h_in.copy_(embedding, non_blocking=True)
        y = self.replay()
        out.copy_(y, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out
