"""Expert-parallel MoE host logic on CPU: two gloo ranks take the experts `expert_partition` gives them, compute the
router-weighted contributions of their own experts with the oracle, exchange with one all-reduce and must reproduce the
unsharded layer.  The partition itself is checked for every world size: disjoint, complete, balanced to within one."""
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
from trellis_serve_b200.kernels.moe import expert_partition
from trellis_serve_b200.runtime import tp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("experts,world", [(256, 8), (256, 2), (10, 4), (7, 7), (33, 8)])
def test_partition_is_disjoint_complete_and_balanced(experts, world):
    shares = [expert_partition(experts, r, world) for r in range(world)]
    flat = [e for s in shares for e in s]
    assert flat == list(range(experts))
    assert max(len(s) for s in shares) - min(len(s) for s in shares) <= 1
    with pytest.raises(ValueError):
        expert_partition(experts, world, world)
    with pytest.raises(ValueError):
        expert_partition(world - 1, 0, world)


def _experts(E, hidden, inter, K):
    def proj(k, n, base):
        return ([seeded_trellis(base + e, k // 16, n // 16, K) for e in range(E)], [seeded_signs(base + 100 + e, k) for e in range(E)],
                [seeded_signs(base + 200 + e, n) for e in range(E)])
    return proj(hidden, inter, 1000), proj(hidden, inter, 2000), proj(inter, hidden, 3000)


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    orc.set_threads(1)
    E, hidden, inter, top_k, K, cb, tokens = 6, 128, 128, 2, 3, 0, 5
    gate, up, down = _experts(E, hidden, inter, K)
    rng = np.random.default_rng(11)                                        # the same tokens and routing on every rank
    x = rng.standard_normal((tokens, hidden)).astype(np.float16)
    ids = np.stack([rng.choice(E, size=top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    w = rng.random((tokens, top_k)).astype(np.float32)
    mine = set(expert_partition(E, rank, world))
    local_ids = np.where(np.isin(ids, list(mine)), ids, -1)                # slots of other ranks' experts add nothing here
    y = torch.from_numpy(orc.np_moe_layer(x, local_ids, w, gate, up, down, K, cb))
    tp.all_reduce_sum(y)
    full = orc.np_moe_layer(x, ids, w, gate, up, down, K, cb)
    assert orc.max_over_rms(y.numpy(), full) < 1e-9
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_layer(tmp_path):
    ctx = mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=False)
    ctx.join(timeout=120)
    for p in ctx.processes:
        if p.is_alive():
            p.kill()
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
