"""Tensor-parallel sharding of EXL3 linears.

The reference refuses tensor parallelism (cuda/src/sglang_exl3/sglang_glue/linear.py:74-75) but its format layer
states the exact slicing rules (core/src/trellis_core/format/geometry.py:47-66): 128-aligned column slices
(q/k/v/gate/up: trellis dim 1, svh; suh whole) and row slices (o/down: trellis dim 0, suh; svh whole; bias on the
first shard only) are complete EXL3 matrices.  This module applies those rules to tensors and adds the one exchange
step the path has: partial outputs of a row-parallel matrix are summed by an all-reduce.

Works on numpy arrays and torch tensors alike (only slicing is used), so the same code serves the CPU tests
(gloo ranks + oracle) and the GPU loader.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..format import MatrixSlice, MatrixSpec, column_slice, even_shard, row_slice


@dataclass
class ShardedLinear:
    trellis: object
    suh: object
    svh: object
    bias: object | None
    k: int
    n: int
    reduce: bool            # True: outputs are partial sums, all-reduce them


def _narrow(t, nr):
    if nr is None or t is None:
        return t
    index = [slice(None)] * nr.dim + [slice(nr.start, nr.start + nr.length)]
    return t[tuple(index)]


def apply_slice(spec: MatrixSpec, sl: MatrixSlice, trellis, suh, svh, bias=None, reduce: bool = False) -> ShardedLinear:
    k, n = sl.sliced_dims(spec)
    b = _narrow(bias, sl.bias) if sl.bias is not None else (bias if sl.keep_bias else None)
    return ShardedLinear(_narrow(trellis, sl.trellis), _narrow(suh, sl.suh), _narrow(svh, sl.svh), b, k, n, reduce)


def column_parallel(spec: MatrixSpec, trellis, suh, svh, tp_size: int, tp_rank: int, bias=None) -> ShardedLinear:
    """Rank's share of an output-split matrix.  No exchange step: every rank owns whole output columns."""
    start, size = even_shard(spec.n, tp_size, tp_rank)
    return apply_slice(spec, column_slice(spec, start, size), trellis, suh, svh, bias, reduce=False)


def row_parallel(spec: MatrixSpec, trellis, suh, svh, tp_size: int, tp_rank: int, bias=None) -> ShardedLinear:
    """Rank's share of an input-split matrix.  Its output is a partial sum over the rank's input rows."""
    start, size = even_shard(spec.k, tp_size, tp_rank)
    return apply_slice(spec, row_slice(spec, start, size), trellis, suh, svh, bias, reduce=tp_size > 1)


def all_reduce_sum(t, group=None):
    """Sum a row-parallel output over the tensor-parallel group (in place).  torch tensors only."""
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, group=group)
    return t
