"""GPU parity of the many-row fused GEMM on the tcgen05 tensor cores (exl3_linear_tc) against the oracle's fp32
forward (relative L2 <= 2e-3, max|d|/rms <= 4e-3: the product is rounded to fp16 before the output rotation, as in
the reference's many-row path, cuda/src/sglang_exl3/runtime/ops.py:36-59) and against the decode kernel."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200.kernels import linear as lin

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a.view(np.int16) if a.dtype == np.uint16 else a)).to(DEV)


@pytest.fixture(autouse=True)
def _default_tiling():
    yield
    lin.set_tc_tiling(-1)
    lin.set_tc_ksplit(0)


# 512 x 128; 256 x 256 (n = 384, 640, 128 have an odd block: narrow); 384 x 128; 512 x 256 on a CTA pair (same condition)
@pytest.mark.parametrize("tiling", [0, 1, 2, 3])
@pytest.mark.parametrize("K,cb,k,n,rows", [(4, 1, 256, 256, 130), (3, 0, 512, 384, 512), (4, 1, 1024, 640, 700),
                                           (5, 2, 256, 128, 33), (2, 0, 384, 256, 1), (8, 1, 256, 256, 1025),
                                           (3, 0, 384, 768, 300), (6, 1, 256, 512, 257), (5, 2, 256, 512, 300),
                                           (7, 2, 1024, 256, 520)])
@pytest.mark.parametrize("ksplit", [0, 1, 3])     # reduction of a tile cut into parts when tiles are few: default, never, at most 3
def test_tensor_core_gemm_matches_the_oracle(K, cb, k, n, rows, tiling, ksplit):
    tr, suh, svh = seeded_trellis(K * 7 + cb, k // 16, n // 16, K), seeded_signs(1, k), seeded_signs(2, n)
    x = np.random.default_rng(rows).standard_normal((rows, k)).astype(np.float16)
    packed = lin.prepare_matrix(_t(tr))
    lin.set_tc_tiling(tiling)
    lin.set_tc_ksplit(ksplit)
    y = lin.run_tc(_t(x), packed, _t(suh).reshape(1, -1), _t(svh), [], cb)
    torch.cuda.synchronize()
    lin.device_error(torch.device(DEV))
    ref = orc.c_linear_forward(x, tr, suh, svh, K, cb)
    got = y.float().cpu().numpy()
    assert orc.rel_norm(got, ref) <= 2e-3, orc.rel_norm(got, ref)
    assert orc.max_over_rms(got, ref) <= 4e-3, orc.max_over_rms(got, ref)


@pytest.mark.parametrize("tiling", [-1, 3])
@pytest.mark.parametrize("ns", [[256, 128], [256, 512]])       # an odd shard boundary forces narrow tiles; even ones pair up
def test_fused_group_and_bf16_through_the_tensor_core_path(ns, tiling):
    K, cb, k, rows = 4, 1, 512, 300
    lin.set_tc_tiling(tiling)
    parts = [(seeded_trellis(80 + i, k // 16, n // 16, K), seeded_signs(81 + i, k), seeded_signs(84 + i, n)) for i, n in enumerate(ns)]
    b, suh_cat, svh_cat, ends = lin.prepare([_t(p[0]) for p in parts], [_t(p[1]) for p in parts], [_t(p[2]) for p in parts])
    x = np.random.default_rng(3).standard_normal((rows, k)).astype(np.float16)
    y = lin.run_tc(_t(x).to(torch.bfloat16), b, suh_cat, svh_cat, ends, cb)
    assert y.dtype == torch.bfloat16
    xb = _t(x).to(torch.bfloat16).to(torch.float16).cpu().numpy()
    col = 0
    for (tr, suh, svh), n in zip(parts, ns):
        ref = orc.c_linear_forward(xb, tr, suh, svh, K, cb)
        assert orc.rel_norm(y[:, col:col + n].float().cpu().numpy(), ref) <= 6e-3          # bf16 output
        col += n
    y16 = lin.run_tc(_t(x), b, suh_cat, svh_cat, ends, cb)
    dec = lin.run(_t(x), b, suh_cat, svh_cat, ends, cb)
    assert orc.rel_norm(y16.float().cpu().numpy(), dec.float().cpu().numpy()) <= 2e-3     # same answer as the decode kernel


@pytest.mark.parametrize("k,n,rows,ksplit", [(2048, 512, 700, 0),        # 4 tiles: every tile cut (no whole ones)
                                             (1024, 10240, 1024, 0),     # 80 tiles on the device's CTA pairs: a whole wave and a cut tail
                                             (1024, 10240, 1000, 2)])    # the same with ragged rows and at most two parts
def test_pair_tiling_with_a_cut_last_wave_matches_the_narrow_tiling(k, n, rows, ksplit):
    K, cb = 3, 0
    gen = torch.Generator(device=DEV)
    gen.manual_seed(k + n)
    from trellis_serve_b200.runtime.layerset import random_packed, random_signs
    w = random_packed(k, n, K, gen, torch.device(DEV))
    suh, svh = random_signs(k, gen, torch.device(DEV), 1), random_signs(n, gen, torch.device(DEV)).view(-1)
    x = torch.randn((rows, k), device=DEV, generator=gen).half()
    lin.set_tc_tiling(0)
    ref = lin.run_tc(x, w, suh, svh, [], cb).float()
    lin.set_tc_tiling(3)
    lin.set_tc_ksplit(ksplit)
    got = lin.run_tc(x, w, suh, svh, [], cb).float()
    again = lin.run_tc(x, w, suh, svh, [], cb).float()
    torch.cuda.synchronize()
    lin.device_error(torch.device(DEV))
    assert torch.equal(got, again)                                   # parts are added in a fixed order
    err = (got - ref).norm() / ref.norm()
    assert err <= 1e-3, float(err)
    assert float((got - ref).abs().max() / ref.pow(2).mean().sqrt()) <= 4e-3


@pytest.mark.parametrize("k,n,rows,K,cb,shards", [(640, 768, 777, 4, 1, 1), (1152, 1280, 1500, 2, 0, 1), (2048, 512, 2049, 5, 2, 1),
                                                  (1024, 1024, 1025, 8, 1, 2), (896, 19200, 1111, 3, 0, 2), (5120, 4352, 700, 7, 2, 2)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_pair_tiling_without_a_cut_has_the_bits_of_the_narrow_tiling(k, n, rows, K, cb, shards, dtype):
    """The pair kernel rotates inside its epilogue; with no tile cut it adds the same products in the same order as the narrow
    kernel followed by the rotation kernel, so ragged rows, shard groups, every family and both output types agree exactly."""
    from trellis_serve_b200.runtime.layerset import random_packed, random_signs
    gen = torch.Generator(device=DEV)
    gen.manual_seed(k + n + rows)
    w = random_packed(k, n, K, gen, torch.device(DEV))
    suh, svh = random_signs(k, gen, torch.device(DEV), shards), random_signs(n, gen, torch.device(DEV)).view(-1)
    ends = [] if shards == 1 else [n // 2]
    x = torch.randn((rows, k), device=DEV, generator=gen).to(dtype)
    lin.set_tc_ksplit(1)
    lin.set_tc_tiling(0)
    ref = lin.run_tc(x, w, suh, svh, ends, cb)
    lin.set_tc_tiling(3)
    got = lin.run_tc(x, w, suh, svh, ends, cb)
    torch.cuda.synchronize()
    lin.device_error(torch.device(DEV))
    assert got.dtype == dtype and torch.equal(got, ref)


def test_pair_tiling_replays_from_a_cuda_graph_with_fresh_input():
    """Cluster launches, the cut last wave and its rotation launch inside one captured graph; replay on new activations."""
    from trellis_serve_b200.runtime.layerset import random_packed, random_signs
    k, n, rows, K, cb = 1024, 10240, 1024, 3, 0
    gen = torch.Generator(device=DEV)
    gen.manual_seed(99)
    w = random_packed(k, n, K, gen, torch.device(DEV))
    suh, svh = random_signs(k, gen, torch.device(DEV), 1), random_signs(n, gen, torch.device(DEV)).view(-1)
    x = torch.randn((rows, k), device=DEV, generator=gen).half()
    out = torch.empty((rows, n), dtype=torch.float16, device=DEV)
    lin.set_tc_tiling(3)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        lin.run_tc(x, w, suh, svh, [], cb, out=out)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        lin.run_tc(x, w, suh, svh, [], cb, out=out)
    x2 = torch.randn((rows, k), device=DEV, generator=gen).half()
    eager = lin.run_tc(x2, w, suh, svh, [], cb).clone()
    x.copy_(x2)
    g.replay()
    torch.cuda.synchronize()
    lin.device_error(torch.device(DEV))
    assert torch.equal(out, eager)
