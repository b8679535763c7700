"""GPU parity of the routed-expert (MoE) EXL3 layer through the C ABI.

Design follows the reference's MoE parity tool (cuda/src/sglang_exl3/tools/moe_parity_sm86.py): the align contract
(:58-73), the layer against a float64 reference of the exact decoded weights (:76-88) under uniform and zipf-skewed
routing (:50-55), and CUDA-graph replay with fresh routing (:107-131).  The float64 reference is the oracle's
np_moe_layer.  Error bars: a layer chains two quantized GEMMs with fp16 intermediates (gate|up, activation, down
outputs), so the bound is looser than the single-GEMM 2e-3: relative L2 <= 3e-3, max|d|/rms <= 8e-3.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200.kernels import moe

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _experts(seed, E, hidden, inter, K, out_scale=1.0):
    """out_scale: magnitude of svh (real checkpoints carry the 1/sqrt(k)-like scale there; +-1 overflows fp16 at
    hidden 2048 with unit-variance codebook values)."""
    def proj(k, n, base):
        tr = [seeded_trellis(base + e, k // 16, n // 16, K) for e in range(E)]
        suh = [seeded_signs(base + 1000 + e, k) for e in range(E)]
        svh = [(seeded_signs(base + 2000 + e, n).astype(np.float32) * out_scale).astype(np.float16) for e in range(E)]
        return tr, suh, svh
    return proj(hidden, inter, seed), proj(hidden, inter, seed + 10000), proj(inter, hidden, seed + 20000)


def _to_dev(p):
    return tuple([torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(DEV) for a in lst] for lst in p)


def _routing(tokens, top_k, E, seed, zipf=False):
    rng = np.random.default_rng(seed)
    if zipf:
        p = 1.0 / np.arange(1, E + 1) ** 1.1
        p = rng.permutation(p / p.sum())
        ids = np.stack([rng.choice(E, size=top_k, replace=False, p=p) for _ in range(tokens)])
    else:
        logits = rng.standard_normal((tokens, E))
        ids = np.argsort(-logits, axis=1)[:, :top_k]
    w = rng.standard_normal((tokens, top_k)).astype(np.float32)
    w = np.exp(w) / np.exp(w).sum(1, keepdims=True)
    return ids.astype(np.int32), w.astype(np.float32)


@pytest.mark.parametrize("tokens,top_k,E", [(1, 8, 256), (64, 8, 256), (7, 2, 8), (33, 4, 16)])
def test_align_contract(tokens, top_k, E):
    ids, _ = _routing(tokens, top_k, E, 1)
    ids[0, 0] = -1 if tokens > 1 else ids[0, 0]                           # an invalid id is dropped, not routed
    sorted_ids, expert_ids, num_post = moe.align(torch.from_numpy(ids).to(DEV), E)
    torch.cuda.synchronize()
    numel, n_post = ids.size, int(num_post.item())
    assert sorted_ids.numel() == moe.sorted_ids_capacity(tokens, top_k, E) and n_post % 8 == 0 and n_post <= sorted_ids.numel()
    s, e, flat = sorted_ids.cpu().numpy(), expert_ids.cpu().numpy(), ids.reshape(-1)
    valid = s[:n_post][s[:n_post] < numel]
    want = np.nonzero((flat >= 0) & (flat < E))[0]
    assert np.array_equal(np.sort(valid), want)                           # every routed slot exactly once
    assert np.all(s[n_post:] == numel) and np.all(s[:n_post][s[:n_post] >= numel] == numel)      # padding = numel
    for i, slot in enumerate(s[:n_post]):
        if slot < numel:
            assert flat[slot] == e[i // 8]                                # block expert ids are right
    assert np.all(e[n_post // 8:] == -1)


@pytest.mark.parametrize("tokens,zipf", [(1, False), (5, False), (20, True)])
@pytest.mark.parametrize("K,cb", [(3, 0), (4, 1), (3, 2)])
def test_layer_matches_the_float64_reference(tokens, zipf, K, cb):
    E, hidden, inter, top_k = 8, 256, 128, 2
    gate, up, down = _experts(100 * K + cb, E, hidden, inter, K)
    pack = moe.prepare(_to_dev(gate), _to_dev(up), _to_dev(down), cb)
    assert (pack.hidden, pack.inter, pack.num_experts, pack.bits) == (hidden, inter, E, K)
    ids, w = _routing(tokens, top_k, E, 7 + tokens, zipf)
    x = np.random.default_rng(tokens).standard_normal((tokens, hidden)).astype(np.float16)
    y = moe.forward(torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), torch.from_numpy(ids).to(DEV), pack)
    torch.cuda.synchronize()
    ref = orc.np_moe_layer(x, ids, w, gate, up, down, K, cb)
    got = y.float().cpu().numpy()
    assert orc.rel_norm(got, ref) <= 3e-3, orc.rel_norm(got, ref)
    assert orc.max_over_rms(got, ref) <= 8e-3, orc.max_over_rms(got, ref)


def test_config_shape_layer_batch_1_and_64():
    """The 256-expert layer's shape scaled in expert count only: hidden 2048, intermediate 512, top-8, K = 3; 16 experts
    keep the float64 reference fast.  Batch 1 and 64."""
    E, hidden, inter, top_k, K, cb = 16, 2048, 512, 8, 3, 0
    gate, up, down = _experts(4242, E, hidden, inter, K, out_scale=1 / 32)
    pack = moe.prepare(_to_dev(gate), _to_dev(up), _to_dev(down), cb)
    for tokens in (1, 64):
        ids, w = _routing(tokens, top_k, E, 300 + tokens)
        x = np.random.default_rng(tokens).standard_normal((tokens, hidden)).astype(np.float16)
        y = moe.forward(torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), torch.from_numpy(ids).to(DEV), pack)
        ref = orc.np_moe_layer(x, ids, w, gate, up, down, K, cb)
        got = y.float().cpu().numpy()
        assert orc.rel_norm(got, ref) <= 3e-3, (tokens, orc.rel_norm(got, ref))


def test_graph_replay_with_fresh_routing_equals_eager_and_is_deterministic():
    E, hidden, inter, top_k, K, cb, tokens = 8, 256, 128, 2, 4, 0, 6
    gate, up, down = _experts(77, E, hidden, inter, K)
    pack = moe.prepare(_to_dev(gate), _to_dev(up), _to_dev(down), cb)
    ids, w = _routing(tokens, top_k, E, 1)
    x = torch.randn((tokens, hidden), device=DEV).half()
    xs, ws, is_ = x.clone(), torch.from_numpy(w).to(DEV), torch.from_numpy(ids).to(DEV)
    first = moe.forward(xs, ws, is_, pack).clone()
    for _ in range(10):
        assert torch.equal(moe.forward(xs, ws, is_, pack), first)
    out = torch.empty_like(first)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        moe.forward(xs, ws, is_, pack, out=out)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        moe.forward(xs, ws, is_, pack, out=out)
    ids2, w2 = _routing(tokens, top_k, E, 2, zipf=True)
    x2 = torch.randn((tokens, hidden), device=DEV).half()
    eager = moe.forward(x2, torch.from_numpy(w2).to(DEV), torch.from_numpy(ids2).to(DEV), pack).clone()
    xs.copy_(x2)
    ws.copy_(torch.from_numpy(w2).to(DEV))
    is_.copy_(torch.from_numpy(ids2).to(DEV))
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)


def test_no_tokens_and_unsupported_packs():
    E, hidden, inter, K = 4, 128, 128, 3
    gate, up, down = _experts(5, E, hidden, inter, K)
    pack = moe.prepare(_to_dev(gate), _to_dev(up), _to_dev(down), 0)
    y = moe.forward(torch.zeros((0, hidden), dtype=torch.float16, device=DEV), torch.zeros((0, 2), device=DEV),
                    torch.zeros((0, 2), dtype=torch.int32, device=DEV), pack)
    assert y.shape == (0, hidden)
    g, u, d = _to_dev(gate), _to_dev(up), _to_dev(down)
    assert moe.supports(g[0], u[0], d[0], 0) == (True, "")
    ok, why = moe.supports(g[0], u[0], d[0][:1] + [torch.zeros((8, 16, 48), dtype=torch.int16, device=DEV)], 0)
    assert not ok and "differ" in why


def _mixed_experts(seed, Ks, hidden, inter):
    """Experts whose bitrate differs (Ks[e] per expert): the three projections of an expert share its K."""
    gate, up, down = ([], [], []), ([], [], []), ([], [], [])
    for e, K in enumerate(Ks):
        g, u, d = _experts(seed + 31 * e, 1, hidden, inter, K)
        for dst, src in ((gate, g), (up, u), (down, d)):
            for j in range(3):
                dst[j].append(src[j][0])
    return gate, up, down


@pytest.mark.parametrize("tokens,zipf", [(1, False), (9, False), (24, True)])
def test_mixed_bitrate_layer_matches_the_float64_reference(tokens, zipf):
    """Mixed-K expert set (the reference's MixedPack): per-class alignment with an expert map, shared slabs, one combine."""
    Ks = [3, 4, 3, 3, 4, 3, 4, 3, 3, 3, 4, 3]
    E, hidden, inter, top_k, cb = len(Ks), 256, 128, 3, 0
    gate, up, down = _mixed_experts(7000, Ks, hidden, inter)
    pack = moe.prepare_mixed(_to_dev(gate), _to_dev(up), _to_dev(down), cb)
    assert pack.bits == [3, 4] and [p.num_experts for p in pack.packs] == [8, 4] and pack.num_experts == E
    assert [m.tolist() for m in pack.expert_ids] == [[e for e in range(E) if Ks[e] == 3], [e for e in range(E) if Ks[e] == 4]]
    ids, w = _routing(tokens, top_k, E, 90 + tokens, zipf)
    x = np.random.default_rng(tokens).standard_normal((tokens, hidden)).astype(np.float16)
    xt, wt, it = torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), torch.from_numpy(ids).to(DEV)
    routings = moe.align_decode(it, pack, tokens, top_k)
    torch.cuda.synchronize()
    flat = ids.reshape(-1)
    for (s, e, n, block), emap in zip(routings, pack.expert_maps):          # each class sees exactly its own slots
        n_post, s_np, m = int(n.item()), s.cpu().numpy(), emap.cpu().numpy()
        valid = s_np[:n_post][s_np[:n_post] < flat.size]
        assert block == 8 and np.array_equal(np.sort(valid), np.nonzero(m[flat] >= 0)[0])
        for i, slot in enumerate(s_np[:n_post]):
            if slot < flat.size:
                assert m[flat[slot]] == e.cpu().numpy()[i // 8]
    y = moe.run_mixed(xt, wt, it, routings, pack)
    torch.cuda.synchronize()
    ref = orc.np_moe_layer(x, ids, w, gate, up, down, Ks, cb)
    got = y.float().cpu().numpy()
    assert orc.rel_norm(got, ref) <= 3e-3, orc.rel_norm(got, ref)
    assert orc.max_over_rms(got, ref) <= 8e-3, orc.max_over_rms(got, ref)
    assert torch.equal(moe.forward_mixed(xt, wt, it, pack), y)              # deterministic, alignment included


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_shares_add_up_to_the_layer(world):
    """Expert parallelism emulated on one device: every rank's pack holds only its experts (slots of the others belong to
    no class and add nothing), the ranks' outputs summed in fp32 are the whole layer."""
    Ks = [3, 4, 3, 3, 4, 3, 4, 3, 3, 3]
    E, hidden, inter, top_k, cb, tokens = len(Ks), 256, 128, 3, 0, 17
    gate, up, down = _mixed_experts(8100, Ks, hidden, inter)
    ids, w = _routing(tokens, top_k, E, 321)
    x = np.random.default_rng(9).standard_normal((tokens, hidden)).astype(np.float16)
    xt, wt, it = torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), torch.from_numpy(ids).to(DEV)
    total = torch.zeros((tokens, hidden), dtype=torch.float32, device=DEV)
    for rank in range(world):
        share = moe.expert_partition(E, rank, world)
        pack = moe.prepare_mixed(_to_dev(gate), _to_dev(up), _to_dev(down), cb, experts=share)
        assert not pack.covers_all and sorted(int(e) for m in pack.expert_ids for e in m.tolist()) == list(share)
        total += moe.forward_expert_parallel(xt, wt, it, pack, reduce=lambda t: t).float()
    ref = orc.np_moe_layer(x, ids, w, gate, up, down, Ks, cb)
    got = total.cpu().numpy()
    assert orc.rel_norm(got, ref) <= 3e-3, orc.rel_norm(got, ref)
    assert orc.max_over_rms(got, ref) <= 8e-3, orc.max_over_rms(got, ref)
