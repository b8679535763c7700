"""GPU parity of the routed-expert layer when experts see many rows each: the grouped tensor-core GEMM on 128-row moe
blocks (`exl3_moe_tc_experts`), reached through `kernels.moe.run_layer`.

The reference serves such batches by growing its moe block with T * top_k / E (cuda/src/sglang_exl3/kernels/marlin_moe.py:52-57)
and checks them with the same float64 layer reference as the decode-sized ones (tools/moe_parity_sm86.py:76-88); so do
these tests, with the oracle's np_moe_layer.  Error bars as in test_gpu_moe.py: relative L2 <= 3e-3, max|d|/rms <= 8e-3.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import exl3_oracle as orc
from test_gpu_moe import _experts, _mixed_experts, _routing, _to_dev
from trellis_serve_b200.kernels import moe

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_layer(pack, x, w, ids, maps=None):
    tokens, top_k = ids.shape
    need = moe.layer_workspace_bytes([p.num_experts for p in pack.packs], pack.hidden, pack.inter, pack.codebook, tokens, top_k)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    xt, wt, it = torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), torch.from_numpy(ids).to(DEV)
    out = torch.empty_like(xt)
    moe.run_layer(xt, wt, it, pack, out, ws, maps)
    torch.cuda.synchronize()
    return out


def _check(got, ref):
    got = got.float().cpu().numpy()
    assert orc.rel_norm(got, ref) <= 3e-3, orc.rel_norm(got, ref)
    assert orc.max_over_rms(got, ref) <= 8e-3, orc.max_over_rms(got, ref)


@pytest.mark.parametrize("tokens,E,zipf", [(300, 8, False), (700, 4, True), (130, 8, True)])
@pytest.mark.parametrize("K,cb", [(3, 0), (4, 1), (3, 2)])
def test_many_rows_per_expert_match_the_float64_reference(tokens, E, zipf, K, cb):
    """75, 350 and 32 rows per expert on average: single blocks with padding, experts of several 128-row blocks (work items of
    up to four blocks, more than one item for the heavy experts under zipf routing) and experts with no rows at all."""
    hidden, inter, top_k = 256, 128, 2
    assert moe.moe_block_size(tokens, top_k, E) == 128
    gate, up, down = _experts(500 * K + cb + E, E, hidden, inter, K, out_scale=1 / 8)
    pack = moe.prepare_mixed(_to_dev(gate), _to_dev(up), _to_dev(down), cb)
    ids, w = _routing(tokens, top_k, E, 11 + tokens, zipf)
    ids[0, 0] = -1                                                             # an invalid id is dropped, not routed
    x = np.random.default_rng(tokens).standard_normal((tokens, hidden)).astype(np.float16)
    _check(_run_layer(pack, x, w, ids), orc.np_moe_layer(x, ids, w, gate, up, down, K, cb))


def test_tensor_core_and_decode_paths_agree_and_bf16_boundary(monkeypatch):
    """The same batch through both paths: they differ only by fp16 roundings of intermediates.  bf16 in / out equals explicit casts."""
    E, hidden, inter, top_k, K, cb, tokens = 8, 512, 256, 2, 4, 1, 200
    gate, up, down = _experts(909, E, hidden, inter, K, out_scale=1 / 16)
    pack = moe.prepare_mixed(_to_dev(gate), _to_dev(up), _to_dev(down), cb)
    ids, w = _routing(tokens, top_k, E, 5)
    x = np.random.default_rng(1).standard_normal((tokens, hidden)).astype(np.float16)
    tc = _run_layer(pack, x, w, ids)
    monkeypatch.setattr(moe, "TC_ROWS_PER_EXPERT", 1 << 30)
    assert moe.moe_block_size(tokens, top_k, E) == 8
    gemv = _run_layer(pack, x, w, ids)
    monkeypatch.undo()
    assert orc.rel_norm(tc.float().cpu().numpy(), gemv.float().cpu().numpy()) <= 2e-3
    _check(tc, orc.np_moe_layer(x, ids, w, gate, up, down, K, cb))
    xb = torch.from_numpy(x).to(DEV).bfloat16()
    need = moe.layer_workspace_bytes([E], hidden, inter, cb, tokens, top_k)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    outb = torch.empty_like(xb)
    moe.run_layer(xb, torch.from_numpy(w).to(DEV), torch.from_numpy(ids).to(DEV), pack, outb, ws)
    via_half = _run_layer(pack, xb.half().cpu().numpy(), w, ids)
    assert torch.equal(outb, via_half.bfloat16())


def test_mixed_bitrate_and_expert_map_with_many_rows():
    """Two bitrate classes, both above the switch; then an engine-style expert map that leaves experts 1 and 6 to another rank:
    their slots add nothing."""
    Ks = [3, 4, 3, 3, 4, 3, 4, 3]
    E, hidden, inter, top_k, cb, tokens = len(Ks), 256, 128, 2, 0, 400
    gate, up, down = _mixed_experts(7100, Ks, hidden, inter)
    for proj in (gate, up, down):
        proj[2][:] = [(s.astype(np.float32) / 8).astype(np.float16) for s in proj[2]]
    pack = moe.prepare_mixed(_to_dev(gate), _to_dev(up), _to_dev(down), cb)
    assert all(moe.moe_block_size(tokens, top_k, p.num_experts) == 128 for p in pack.packs)
    ids, w = _routing(tokens, top_k, E, 77, zipf=True)
    x = np.random.default_rng(2).standard_normal((tokens, hidden)).astype(np.float16)
    _check(_run_layer(pack, x, w, ids), orc.np_moe_layer(x, ids, w, gate, up, down, Ks, cb))
    held = [e for e in range(E) if e not in (1, 6)]
    maps = []
    for m in pack.expert_maps:
        m2 = m.clone()
        m2[[1, 6]] = -1
        maps.append(m2)
    ids_held = np.where(np.isin(ids, held), ids, -1)
    _check(_run_layer(pack, x, w, ids, maps), orc.np_moe_layer(x, ids_held, w, gate, up, down, Ks, cb))


def test_graph_replay_with_fresh_routing_allocates_nothing():
    E, hidden, inter, top_k, K, cb, tokens = 4, 256, 128, 2, 3, 0, 160
    gate, up, down = _experts(31, E, hidden, inter, K, out_scale=1 / 8)
    pack = moe.prepare_mixed(_to_dev(gate), _to_dev(up), _to_dev(down), cb)
    need = moe.layer_workspace_bytes([E], hidden, inter, cb, tokens, top_k)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    ids, w = _routing(tokens, top_k, E, 1)
    xs = torch.randn((tokens, hidden), device=DEV).half()
    wt, it = torch.from_numpy(w).to(DEV), torch.from_numpy(ids).to(DEV)
    out, out2 = torch.empty_like(xs), torch.empty_like(xs)
    moe.run_layer(xs, wt, it, pack, out, ws)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    moe.run_layer(xs, wt, it, pack, out2, ws)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before and torch.equal(out, out2)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        moe.run_layer(xs, wt, it, pack, out, ws)
    ids2, w2 = _routing(tokens, top_k, E, 2, zipf=True)
    x2 = torch.randn((tokens, hidden), device=DEV).half()
    moe.run_layer(x2, torch.from_numpy(w2).to(DEV), torch.from_numpy(ids2).to(DEV), pack, out2, ws)
    xs.copy_(x2)
    wt.copy_(torch.from_numpy(w2).to(DEV))
    it.copy_(torch.from_numpy(ids2).to(DEV))
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
