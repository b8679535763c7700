"""Two-GPU test of the one-shot peer-memory all-reduce (skipped with fewer than two devices): every rank must get
exactly the fp32 rank-order sum of all ranks' inputs, call after call, also under CUDA-graph replay."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from trellis_serve_b200.runtime.allreduce import PeerAllReduce
    ar = PeerAllReduce(dev, 16 * 5120)
    gen = torch.Generator(device=dev)
    for call, (rows, dtype) in enumerate([(1, torch.float16), (3, torch.float16), (16, torch.bfloat16), (1, torch.float16)]):
        gen.manual_seed(100 * call + rank)
        x = torch.randn((rows, 5120), device=dev, generator=gen).to(dtype)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        want = sum(p.float() for p in parts).to(dtype)                      # fp32 sum in rank order, one rounding
        got = ar(x.clone())
        torch.cuda.synchronize()
        ar.check()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (rank, call)
    # The exchange fused into the row-parallel linear gives the bits of linear followed by the all-reduce; the two kinds
    # of call share regions and the call counter, so they are interleaved here.  Shapes: several column blocks per CTA
    # range and ranges that share blocks; 1, 2 (in-kernel rotation), 5 and 16 rows; fp16 and bf16.
    from trellis_serve_b200.kernels import linear as lin
    from trellis_serve_b200.runtime.layerset import random_packed, random_signs
    for call, (rows, k, n, K, dtype) in enumerate([(1, 1024, 5120, 3, torch.float16), (2, 512, 5120, 4, torch.bfloat16),
                                                   (5, 2176, 5120, 3, torch.float16), (16, 640, 5120, 2, torch.float16),
                                                   (1, 2176, 5120, 3, torch.float16)]):
        gen.manual_seed(7000 + 10 * call + rank)
        w = random_packed(k, n, K, gen, dev)
        suh, svh = random_signs(k, gen, dev, 1), (random_signs(n, gen, dev).view(-1) / 16).half()
        x = torch.randn((rows, k), device=dev, generator=gen).to(dtype)
        want = ar(lin.run(x, w, suh, svh, [], 0))
        got = lin.run(x, w, suh, svh, [], 0, exchange=ar)
        torch.cuda.synchronize()
        ar.check()
        lin.device_error(dev)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (rank, "fused", call)
    # The residual epilogue behind the fused exchange (one and two rows, a pre-rotated input and a gate | up input): the new
    # stream is round(sum over ranks of y + z), the same bits on every rank, and its sums of squares are those of what was stored.
    for call, (rows, k, n, K, dtype, glu) in enumerate([(1, 1024, 5120, 3, torch.float16, False), (2, 512, 5120, 4, torch.bfloat16, True),
                                                        (1, 640, 5120, 3, torch.bfloat16, True), (2, 2176, 5120, 3, torch.float16, False)]):
        gen.manual_seed(9000 + 10 * call + rank)
        w = random_packed(k, n, K, gen, dev)
        suh, svh = random_signs(k, gen, dev, 1), (random_signs(n, gen, dev).view(-1) / 16).half()
        ws = torch.zeros(lin.workspace_bytes(16, k, n, 1), dtype=torch.uint8, device=dev)
        gen.manual_seed(9500 + call)                                        # the residual stream is replicated: same on every rank
        z = torch.randn((rows, n), device=dev, generator=gen).to(dtype)
        gen.manual_seed(9700 + 10 * call + rank)
        y, z2 = torch.empty((rows, n), dtype=dtype, device=dev), torch.empty((rows, n), dtype=dtype, device=dev)
        ssq = torch.zeros((rows, n // 128), dtype=torch.float32, device=dev)
        if glu:
            gu = torch.randn((rows, 2 * k), device=dev, generator=gen).to(dtype)
            want_y = ar(lin.run_glu(gu, w, suh.view(-1), svh, 0, torch.empty_like(y), ws))
            lin.run_glu(gu, w, suh.view(-1), svh, 0, y, ws, exchange=ar, residual=(z, z2, ssq))
        else:
            x = torch.randn((rows, k), device=dev, generator=gen).to(dtype)
            want_y = ar(lin.run(x, w, suh, svh, [], 0))
            lin.rotate_fragments(x, suh, 0, ws)
            lin.run_prerotated(rows, w, svh, [], 0, y, ws, exchange=ar, residual=(z, z2, ssq))
        torch.cuda.synchronize()
        ar.check()
        lin.device_error(dev)
        assert torch.equal(y.view(torch.int16), want_y.view(torch.int16)), (rank, "residual y", call)
        want_z = (want_y.float() + z.float()).to(dtype)
        assert torch.equal(z2.view(torch.int16), want_z.view(torch.int16)), (rank, "residual stream", call)
        want_ssq = want_z.float().view(rows, n // 128, 128).pow(2).sum(-1)
        assert float(((ssq - want_ssq).abs() / want_ssq).max()) <= 1e-5, (rank, "sums of squares", call)
        both = [torch.empty_like(z2) for _ in range(world)]
        dist.all_gather(both, z2)
        assert all(torch.equal(b.view(torch.int16), both[0].view(torch.int16)) for b in both), (rank, "replicated stream", call)
    # CUDA-graph replay: the call counter lives on the device, so a replay is a new call
    buf = torch.zeros((1, 5120), dtype=torch.float16, device=dev)
    src = torch.zeros_like(buf)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        buf.copy_(src)
        ar(buf)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        buf.copy_(src)
        ar(buf)
    for it in range(3):
        src.fill_(float(rank + 1 + it))
        g.replay()
        torch.cuda.synchronize()
        assert torch.all(buf == float(sum(r + 1 + it for r in range(world)))), (rank, it)
    ar.check()
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_get_the_same_exact_sum(tmp_path):
    ctx = mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=False)
    ctx.join(timeout=150)
    for p in ctx.processes:
        if p.is_alive():
            p.kill()
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
