"""GPU parity at the full sizes of the 27B-shape layer set, through the C ABI, against the CPU oracle.

The small-shape files prove the arithmetic; this one proves the schedules that only real shapes reach: fused groups of
272 column blocks, 136 reduction blocks per column (the longest fp32 accumulation and the most split-k hand-overs),
two-wave tile lists of the tensor-core kernel, 256 experts, and the row ladder of the reference's environment diff
(cuda/src/sglang_exl3/parity/l1_linear.py:24-25), which crosses the decode / tensor-core switch and the 16-row chunk seam.
Bounds as in the small-shape files: max|d|/rms(ref) <= 2e-3 and relative L2 <= 2e-3 on the fp32 accumulators of the decode
kernel, the fp16 result equal to those rounded once; relative L2 <= 2e-3 and max|d|/rms <= 4e-3 for the tensor-core kernel.
"""
from __future__ import annotations

import hashlib

import numpy as np
import pytest
import torch

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200.kernels import linear as lin
from trellis_serve_b200.kernels import moe

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-3

HIDDEN, KV, FFN = 5120, 1024, 17408
GROUPS = {                       # name -> (k, [n per matrix])
    "qkv": (HIDDEN, [HIDDEN, KV, KV]),
    "o": (HIDDEN, [HIDDEN]),
    "gate_up": (HIDDEN, [FFN, FFN]),
    "down": (FFN, [HIDDEN]),
}


def _t(a: np.ndarray) -> torch.Tensor:
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _group(seed: int, name: str, K: int, out_scale: float = 1.0):
    k, ns = GROUPS[name]
    parts = []
    for i, n in enumerate(ns):
        svh = (seeded_signs(seed + 20 + i, n).astype(np.float32) * out_scale).astype(np.float16)
        parts.append((seeded_trellis(seed + i, k // 16, n // 16, K), seeded_signs(seed + 10 + i, k), svh))
    return k, ns, parts


def _prepare(parts):
    return lin.prepare([_t(p[0]) for p in parts], [_t(p[1]) for p in parts], [_t(p[2]) for p in parts])


# ------------------------------------------------------------------------------------------------ decode kernel

@pytest.mark.parametrize("rows", [1, 4, 16])
@pytest.mark.parametrize("name", ["gate_up", "down", "qkv", "o"])
def test_decode_forward_at_the_27b_shapes(name, rows):
    """K = 3, 3INST, batch 1 / 4 / 16: every output column of every matrix of the group against the oracle."""
    K, cb = 3, 0
    k, ns, parts = _group(4000 + 37 * len(name), name, K, out_scale=1 / 64)
    b, suh_cat, svh_cat, ends = _prepare(parts)
    x = np.random.default_rng(rows + k).standard_normal((rows, k)).astype(np.float16)
    xs = _t(x)
    y32 = torch.empty((rows, sum(ns)), dtype=torch.float32, device=DEV)
    lin.run(xs, b, suh_cat, svh_cat, ends, cb, out=y32)
    y16 = lin.run(xs, b, suh_cat, svh_cat, ends, cb)
    torch.cuda.synchronize()
    lin.device_error(torch.device(DEV))
    assert torch.equal(y16, y32.to(torch.float16))
    got32, got16, col = y32.cpu().numpy(), y16.float().cpu().numpy(), 0
    for (tr, suh, svh), n in zip(parts, ns):
        ref = orc.c_linear_forward(x, tr, suh, svh, K, cb)
        assert orc.max_over_rms(got32[:, col:col + n], ref) <= TOL, (name, rows, orc.max_over_rms(got32[:, col:col + n], ref))
        assert orc.rel_norm(got32[:, col:col + n], ref) <= TOL
        assert orc.rel_norm(got16[:, col:col + n], ref) <= TOL
        col += n


@pytest.mark.parametrize("K", range(2, 9))
def test_decode_is_bit_exact_at_the_down_projection_shape(K):
    """17408 x 5120, every bit rate: all 89 million decoded weights equal the oracle's."""
    cb = 0
    tr = seeded_trellis(5000 + K, FFN // 16, HIDDEN // 16, K)
    w = lin.reconstruct_packed(lin.prepare_matrix(_t(tr)), cb)
    got = _bits16(w)
    del w
    assert np.array_equal(got, orc.c_reconstruct(tr, K, cb).view(np.uint16))


# ------------------------------------------------------------------------------------------------ tensor-core kernel

@pytest.mark.parametrize("name", ["o", "down", "qkv", "gate_up"])
def test_tensor_core_forward_at_the_27b_shapes_2048_rows(name):
    """rows = 2048, K = 4, MCG: all columns of 96 rows spread over every row tile (the oracle's fp32 product of all 2048 rows
    would take minutes; an output row depends on its own input row only)."""
    K, cb, rows = 4, 1, 2048
    k, ns, parts = _group(6000 + 41 * len(name), name, K, out_scale=1 / 64)
    b, suh_cat, svh_cat, ends = _prepare(parts)
    x = np.random.default_rng(k + len(name)).standard_normal((rows, k)).astype(np.float16)
    y = lin.run_tc(_t(x), b, suh_cat, svh_cat, ends, cb)
    torch.cuda.synchronize()
    lin.device_error(torch.device(DEV))
    pick = np.unique(np.concatenate([np.arange(0, rows, 23), [127, 128, 383, 384, 511, 512, 1023, 1535, 1536, 2047]]))
    got, col = y[torch.from_numpy(pick).to(DEV)].float().cpu().numpy(), 0
    for (tr, suh, svh), n in zip(parts, ns):
        ref = orc.c_linear_forward(x[pick], tr, suh, svh, K, cb)
        assert orc.rel_norm(got[:, col:col + n], ref) <= 2e-3, (name, orc.rel_norm(got[:, col:col + n], ref))
        assert orc.max_over_rms(got[:, col:col + n], ref) <= 4e-3, (name, orc.max_over_rms(got[:, col:col + n], ref))
        col += n


# ------------------------------------------------------------------------------------------------ the operator's row ladder

def _sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()[:16]


def test_row_ladder_through_the_operator():
    """Rows 1, 2, 3, 8, 16, 17, 64, 144, 145, 512 (l1_linear.py:24) through `torch.ops.exl3_b200.linear` on one q|k|v-like
    group: each against the oracle, and hashed twice to show the same bits run to run, as the reference's environment diff
    does with its content hashes (l1_linear.py:39-63)."""
    from trellis_serve_b200.runtime import ops
    K, cb, k, ns = 4, 1, 1024, [768, 256]
    parts = [(seeded_trellis(7000 + i, k // 16, n // 16, K), seeded_signs(7010 + i, k),
              (seeded_signs(7020 + i, n).astype(np.float32) / 32).astype(np.float16)) for i, n in enumerate(ns)]
    b, suh_cat, svh_cat, ends = _prepare(parts)
    gen = np.random.default_rng(1234)
    for rows in (1, 2, 3, 8, 16, 17, 64, 144, 145, 512):
        x = (gen.standard_normal((rows, k)) * 0.5).astype(np.float16)
        xs = _t(x)
        y = ops.linear(xs, [], [], [], [], [], 0, [b, suh_cat, svh_cat], ends, [cb] * len(ns), ns)
        again = ops.linear(xs, [], [], [], [], [], 0, [b, suh_cat, svh_cat], ends, [cb] * len(ns), ns)
        assert y.shape == (rows, sum(ns)) and _sha(y) == _sha(again)
        got, col = y.float().cpu().numpy(), 0
        for (tr, suh, svh), n in zip(parts, ns):
            ref = orc.c_linear_forward(x, tr, suh, svh, K, cb)
            assert orc.rel_norm(got[:, col:col + n], ref) <= 2e-3, (rows, orc.rel_norm(got[:, col:col + n], ref))
            assert orc.max_over_rms(got[:, col:col + n], ref) <= 4e-3, (rows, orc.max_over_rms(got[:, col:col + n], ref))
            col += n


# ------------------------------------------------------------------------------------------------ MoE at 256 experts

def _experts(seed, E, hidden, inter, K, out_scale):
    def proj(k, n, base):
        tr = [seeded_trellis(base + e, k // 16, n // 16, K) for e in range(E)]
        suh = [seeded_signs(base + 1000 + e, k) for e in range(E)]
        svh = [(seeded_signs(base + 2000 + e, n).astype(np.float32) * out_scale).astype(np.float16) for e in range(E)]
        return tr, suh, svh
    return proj(hidden, inter, seed), proj(hidden, inter, seed + 10000), proj(inter, hidden, seed + 20000)


def test_moe_layer_with_256_experts_batch_1_and_64():
    """hidden 2048, 256 experts, intermediate 512, top-8 by softmax over N(0,1) router logits, K = 3, 3INST; 1 and 64 tokens
    against the float64 layer (which decodes only the routed experts)."""
    E, hidden, inter, top_k, K, cb = 256, 2048, 512, 8, 3, 0
    gate, up, down = _experts(9000, E, hidden, inter, K, out_scale=1 / 32)
    dev = lambda p: tuple([_t(a) for a in lst] for lst in p)
    pack = moe.prepare(dev(gate), dev(up), dev(down), cb)
    for tokens in (1, 64):
        rng = np.random.default_rng(300 + tokens)
        logits = rng.standard_normal((tokens, E))
        prob = np.exp(logits) / np.exp(logits).sum(1, keepdims=True)
        ids = np.argsort(-prob, axis=1)[:, :top_k].astype(np.int32)
        w = np.take_along_axis(prob, ids, axis=1).astype(np.float32)
        x = rng.standard_normal((tokens, hidden)).astype(np.float16)
        y = moe.forward(_t(x), _t(w), _t(ids), pack)
        torch.cuda.synchronize()
        ref = orc.np_moe_layer(x, ids, w, gate, up, down, K, cb, reconstruct=orc.c_reconstruct)
        got = y.float().cpu().numpy()
        assert orc.rel_norm(got, ref) <= 3e-3, (tokens, orc.rel_norm(got, ref))
        assert orc.max_over_rms(got, ref) <= 8e-3, (tokens, orc.max_over_rms(got, ref))
