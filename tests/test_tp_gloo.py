"""Tensor-parallel host logic on CPU: two gloo ranks shard a q-like (column-parallel) and an o-like (row-parallel)
EXL3 matrix with the slicing rules, run their shards through the oracle, exchange with one all-reduce and must
reproduce the unsharded forward.  Also covers a rank that never joins: the others get a time-out error, not a hang."""
from __future__ import annotations

import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200.format import TensorInfo, build_matrix_spec
from trellis_serve_b200.runtime import tp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spec(key, k, n, K):
    return build_matrix_spec(key, {"trellis": TensorInfo(f"{key}.trellis", "I16", (k // 16, n // 16, 16 * K)),
                                   "suh": TensorInfo(f"{key}.suh", "F16", (k,)), "svh": TensorInfo(f"{key}.svh", "F16", (n,))})


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    orc.set_threads(1)
    K, cb, hidden, q_out = 3, 0, 512, 256
    x = np.random.default_rng(5).standard_normal((2, hidden)).astype(np.float16)
    # column parallel (q): every rank gets whole columns, results are concatenated
    tq, sq, vq = seeded_trellis(1, hidden // 16, q_out // 16, K), seeded_signs(2, hidden), seeded_signs(3, q_out)
    sh = tp.column_parallel(_spec("q", hidden, q_out, K), tq, sq, vq, world, rank)
    assert (sh.k, sh.n, sh.reduce) == (hidden, q_out // world, False)
    yq = torch.from_numpy(orc.c_linear_forward(x, np.ascontiguousarray(sh.trellis), sh.suh, np.ascontiguousarray(sh.svh), K, cb))
    parts = [torch.empty_like(yq) for _ in range(world)]
    dist.all_gather(parts, yq)
    full_q = orc.c_linear_forward(x, tq, sq, vq, K, cb)
    assert np.array_equal(torch.cat(parts, dim=1).numpy(), full_q)              # exact: same arithmetic per column
    # row parallel (o): every rank multiplies its slice of the input, partial sums are all-reduced
    a = np.random.default_rng(6).standard_normal((2, q_out)).astype(np.float16)
    to, so, vo = seeded_trellis(4, q_out // 16, hidden // 16, K), seeded_signs(5, q_out), seeded_signs(6, hidden)
    sh = tp.row_parallel(_spec("o", q_out, hidden, K), to, so, vo, world, rank)
    assert (sh.k, sh.n, sh.reduce) == (q_out // world, hidden, True)
    start = rank * sh.k
    yo = torch.from_numpy(orc.c_linear_forward(np.ascontiguousarray(a[:, start:start + sh.k]), np.ascontiguousarray(sh.trellis),
                                               np.ascontiguousarray(sh.suh), sh.svh, K, cb))
    tp.all_reduce_sum(yo)
    full_o = orc.c_linear_forward(a, to, so, vo, K, cb)
    assert orc.max_over_rms(yo.numpy(), full_o) < 1e-5
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_forward(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def _lonely(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
        open(os.path.join(out_dir, "joined"), "w").write("unexpected")
    except Exception as e:                                        # the missing rank shows up as an error, not a hang
        open(os.path.join(out_dir, "timeout"), "w").write(type(e).__name__)


def test_a_rank_that_never_joins_is_a_timeout_not_a_hang(tmp_path):
    mp.spawn(_lonely, args=(2, _free_port(), str(tmp_path)), nprocs=1, join=True)      # rank 1 is never started
    assert os.listdir(tmp_path) == ["timeout"]
