"""The `linear` operator: one opaque op per fused EXL3 group with every row-count branch, dtype cast, pad and trim
inside, as the reference's cuda/src/sglang_exl3/runtime/ops.py:62-137 (0xSero/trellis-serve) does for its engines.

Same schema as the reference's custom op (ops.py:133):

    linear(Tensor x, Tensor[] trellis, Tensor[] suh, Tensor[] svh, Tensor[] dense, Tensor[] sliced, int sliced_min_rows,
           Tensor[] marlin_w, int[] marlin_ends, int[] codebooks, int[] out_widths) -> Tensor

registered as `torch.ops.exl3_b200.linear`, with a fake (meta) implementation so tracing compilers see only shapes.
`marlin_w` carries the output of `kernels.linear.prepare`: [packed, suh_cat, svh_cat]; `marlin_ends` its shard ends.
`trellis`, `suh`, `svh` (the stored tensors) are optional here: the resident layout alone serves every path.
`dense` may hold resident decoded fp16 weights per matrix; `sliced` is accepted for schema compatibility and unused.

Dispatch (there is a single backend, so the reference's ladder, ops.py:79-95, collapses to two paths):

  few rows                  fused decode kernel (weights streamed once per 16 rows)
  many rows                 many-row path: the fused tcgen05 kernel (`kernels.linear.run_tc`: weights decoded once per
                            512 rows into the tensor-core operand); when resident decoded weights are passed in `dense`,
                            `dense_group` instead (batched input rotation, library fp16 GEMM on the resident weight,
                            output rotation), which is the reference's many-row sequence

x may have any leading dims; a last dim narrower than the stored (128-padded) k is zero-padded (ops.py:98-99) and
stored output columns beyond the true `out_widths` are dropped (ops.py:122-124).  fp16 / bf16 go through as they are;
any other dtype is computed in fp16 and cast back.
"""
from __future__ import annotations

import os

import torch

from .._lib import sm_count as lib_sm_count
from ..kernels import linear as lin

_lib = torch.library.Library("exl3_b200", "FRAGMENT")       # must stay alive at module scope

# Row count from which the many-row path is taken; 0 = decide per call with `prefers_decode` (the crossover depends on the
# shape and, since narrow outputs split their reduction over the idle SMs, lies at 17 rows for the 27B-shape groups).
DENSE_ROWS = int(os.environ.get("EXL3_B200_DENSE_ROWS", "0"))


def prefers_decode(rows: int, k: int, n_total: int, sms: int = 148) -> bool:
    """Cost model fitted to measurements on B200 (microseconds); `sms` is the device's multiprocessor count.  The decode kernel streams the weights once per 16 rows:
    ~14 + 0.38 per million weights for a full chunk, ~0.8 of that for a last chunk of up to 8 rows.  The tensor-core kernel
    works through its tiles in waves over the SMs at ~1.1 per 64-deep reduction block (~1.6 for the 512-row tiles used above
    256 rows); when the tiles are fewer than the SMs the reduction of each is cut into up to 8 parts on CTAs of their own;
    ~12 more for the two rotation launches, ~8 for adding the parts."""
    mw = k * n_total / 1e6
    chunk = 14.0 + 0.38 * mw
    full, rem = divmod(rows, 16)
    decode = full * chunk + (0.0 if rem == 0 else chunk * (0.8 if rem <= 8 else 1.0))
    if rows <= 256:
        tiles, per_block = -(-rows // 256) * max(n_total // 256, 1), 1.1
    else:
        tiles, per_block = -(-rows // 512) * (n_total // 128), 1.6
    parts = max(1, min(8, sms // max(tiles, 1), k // 64))
    tensor = -(-tiles // sms) * (k / 64) / parts * per_block + 12.0 + (8.0 if parts > 1 else 0.0) + 0.08 * min(rows, 256)
    return decode <= tensor
# "tc": fused tcgen05 kernel; "library": decode to fp16 + library GEMM (the reference's sequence), for comparisons.
PREFILL = os.environ.get("EXL3_B200_PREFILL", "tc")


def dense_group(x: torch.Tensor, packed: torch.Tensor, suh_cat: torch.Tensor, svh_cat: torch.Tensor, shard_ends: list[int],
                codebook: int, out: torch.Tensor, weights: list[torch.Tensor] | None = None) -> torch.Tensor:
    """Many-row (prefill) path of a fused group, the reference's `dense_group` (ops.py:36-59): ONE batched input
    rotation for all matrices, per matrix the decoded fp16 weight (resident `weights[i]`, or decoded now from the
    resident layout) times the rotated rows in an fp16 GEMM with fp32 accumulation, and an output rotation written
    straight into the matrix's column span of `out` in out's dtype."""
    rows = x.shape[0]
    xh = lin.had_in_group(x, suh_cat)
    bounds = [0, *shard_ends, svh_cat.shape[0]]
    for i, (a, b) in enumerate(zip(bounds[:-1], bounds[1:])):
        w = weights[i] if weights is not None else lin.reconstruct_packed(packed[a // 128:b // 128], codebook)
        y = torch.mm(xh[i * rows:(i + 1) * rows], w)
        del w
        lin.had_out_into(y, svh_cat[a:b], out, a)
    return out


def _linear(x: torch.Tensor, trellis: list[torch.Tensor], suh: list[torch.Tensor], svh: list[torch.Tensor],
            dense: list[torch.Tensor], sliced: list[torch.Tensor], sliced_min_rows: int, marlin_w: list[torch.Tensor],
            marlin_ends: list[int], codebooks: list[int], out_widths: list[int]) -> torch.Tensor:
    if len(marlin_w) != 3:
        raise RuntimeError("marlin_w must be [packed, suh_cat, svh_cat] from kernels.linear.prepare")
    if len(set(codebooks)) != 1:
        raise RuntimeError("one codebook per fused group")
    packed, suh_cat, svh_cat = marlin_w
    ends = list(marlin_ends)
    k, n_total = packed.shape[1] * 128, packed.shape[0] * 128
    rows = x.reshape(-1, x.shape[-1])
    h = rows if rows.dtype in (torch.float16, torch.bfloat16) else rows.to(torch.float16)
    if h.shape[1] > k:
        raise RuntimeError(f"input width {h.shape[1]} exceeds the stored width {k}")
    if h.shape[1] < k:                                   # stored input width is padded to 128
        h = torch.nn.functional.pad(h, (0, k - h.shape[1]))
    h = h.contiguous()
    sms = lib_sm_count(h.device.index if h.device.index is not None else torch.cuda.current_device())
    if (h.shape[0] < DENSE_ROWS) if DENSE_ROWS > 0 else prefers_decode(h.shape[0], k, n_total, sms):
        y = lin.run(h, packed, suh_cat, svh_cat, ends, codebooks[0])
    elif dense or PREFILL == "library":
        y = torch.empty((h.shape[0], n_total), dtype=h.dtype, device=h.device)
        dense_group(h, packed, suh_cat, svh_cat, ends, codebooks[0], y, list(dense) if dense else None)
    else:
        y = lin.run_tc(h, packed, suh_cat, svh_cat, ends, codebooks[0])
    bounds = [0, *ends, n_total]
    stored = [b - a for a, b in zip(bounds[:-1], bounds[1:])]
    if any(w > s for w, s in zip(out_widths, stored)):   # logical widths beyond the stored ones read as zeros (ops.py:117-121)
        padded = torch.zeros((y.shape[0], sum(out_widths)), dtype=y.dtype, device=y.device)
        col = 0
        for a, w, s in zip(bounds[:-1], out_widths, stored):
            keep = min(w, s)
            padded[:, col:col + keep] = y[:, a:a + keep]
            col += w
        y = padded
    elif list(out_widths) != stored:                     # stored output columns beyond the true width are dropped
        y = torch.cat([y[:, a:a + w] for a, w in zip(bounds[:-1], out_widths)], dim=1)
    return y.to(x.dtype).view(*x.shape[:-1], y.shape[1])


def _linear_fake(x, trellis, suh, svh, dense, sliced, sliced_min_rows, marlin_w, marlin_ends, codebooks, out_widths):
    return x.new_empty((*x.shape[:-1], sum(out_widths)))


_lib.define("linear(Tensor x, Tensor[] trellis, Tensor[] suh, Tensor[] svh, Tensor[] dense, Tensor[] sliced, int sliced_min_rows, "
            "Tensor[] marlin_w, int[] marlin_ends, int[] codebooks, int[] out_widths) -> Tensor")
_lib.impl("linear", _linear, "CUDA")
torch.library.register_fake("exl3_b200::linear", _linear_fake, lib=_lib)

linear = torch.ops.exl3_b200.linear
