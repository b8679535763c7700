"""The `linear` operator (runtime/ops.py): shape inference without a GPU, and on a GPU both row-count paths, the
pad / trim rules (reference ops.py:98-99, :122-124), leading dims, dtype handling, and the prefill path against the
oracle and against the decode path (the reference checks prefill == explicit path at 96 rows,
cuda/src/sglang_exl3/parity/marlin_parity.py:130-146)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200.runtime import ops

DEV = "cuda:0"


def test_fake_implementation_infers_shapes_without_a_gpu():
    x = torch.empty((2, 3, 500), device="meta", dtype=torch.bfloat16)
    packed = torch.empty((5, 4, 8, 2, 3, 32), device="meta", dtype=torch.int32)
    y = ops.linear(x, [], [], [], [], [], 0, [packed, packed, packed], [384], [0, 0], [380, 250])
    assert y.shape == (2, 3, 630) and y.dtype == torch.bfloat16


def _group(K, cb, k, ns, seed):
    from trellis_serve_b200.kernels import linear as lin
    parts = []
    for i, n in enumerate(ns):
        parts.append((seeded_trellis(seed + i, k // 16, n // 16, K), seeded_signs(seed + 10 + i, k), seeded_signs(seed + 20 + i, n)))
    dev = [[torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(DEV) for a in p] for p in parts]
    b, suh_cat, svh_cat, ends = lin.prepare([d[0] for d in dev], [d[1] for d in dev], [d[2] for d in dev])
    return parts, [b, suh_cat, svh_cat], ends


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 16, 40, 300])
def test_both_paths_match_the_oracle(rows):
    K, cb, k, ns = 4, 1, 512, [256, 128]
    parts, w, ends = _group(K, cb, k, ns, 31)
    x = np.random.default_rng(rows).standard_normal((rows, k)).astype(np.float16)
    y = ops.linear(torch.from_numpy(x).to(DEV), [], [], [], [], [], 0, w, ends, [cb, cb], ns).float().cpu().numpy()
    col = 0
    for (tr, suh, svh), n in zip(parts, ns):
        ref = orc.c_linear_forward(x, tr, suh, svh, K, cb)
        assert orc.rel_norm(y[:, col:col + n], ref) <= 2e-3, (rows, orc.rel_norm(y[:, col:col + n], ref))
        col += n


@pytest.mark.gpu
def test_prefill_path_agrees_with_the_decode_path(monkeypatch):
    K, cb, k, ns = 3, 0, 1024, [384]
    parts, w, ends = _group(K, cb, k, ns, 47)
    x = torch.from_numpy(np.random.default_rng(1).standard_normal((96, k)).astype(np.float16)).to(DEV)
    monkeypatch.setattr(ops, "DENSE_ROWS", 10 ** 9)
    decode = ops.linear(x, [], [], [], [], [], 0, w, ends, [cb], ns).float()
    monkeypatch.setattr(ops, "DENSE_ROWS", 1)
    fused = ops.linear(x, [], [], [], [], [], 0, w, ends, [cb], ns).float()           # tcgen05 kernel
    assert orc.rel_norm(fused.cpu().numpy(), decode.cpu().numpy()) <= 2e-3
    monkeypatch.setattr(ops, "PREFILL", "library")
    prefill = ops.linear(x, [], [], [], [], [], 0, w, ends, [cb], ns).float()         # decode + library GEMM
    assert orc.rel_norm(prefill.cpu().numpy(), decode.cpu().numpy()) <= 2e-3
    from trellis_serve_b200.kernels import linear as lin
    resident = [lin.reconstruct_packed(w[0], cb)]
    cached = ops.linear(x, [], [], [], resident, [], 0, w, ends, [cb], ns).float()
    assert torch.equal(cached, prefill)                                   # resident decoded weight: same bits


@pytest.mark.gpu
def test_pad_trim_leading_dims_and_dtypes():
    K, cb, k, ns = 4, 0, 256, [256, 128]
    parts, w, ends = _group(K, cb, k, ns, 59)
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 3, 250)).astype(np.float32)               # narrower than the stored 256, fp32 caller
    y = ops.linear(torch.from_numpy(x).to(DEV), [], [], [], [], [], 0, w, ends, [cb, cb], [250, 100])
    assert y.shape == (2, 3, 350) and y.dtype == torch.float32
    xp = np.zeros((6, k), dtype=np.float16)
    xp[:, :250] = x.reshape(6, 250).astype(np.float16)
    refs = [orc.c_linear_forward(xp, *p, K, cb) for p in parts]
    want = np.concatenate([refs[0][:, :250], refs[1][:, :100]], axis=1)
    assert orc.rel_norm(y.reshape(6, 350).cpu().numpy(), want) <= 2e-3
    yb = ops.linear(torch.from_numpy(xp).to(DEV).to(torch.bfloat16), [], [], [], [], [], 0, w, ends, [cb, cb], ns)
    assert yb.dtype == torch.bfloat16 and yb.shape == (6, 384)
    # logical widths beyond the stored ones: the extra columns read as zeros (reference ops.py:101-102, :117-121)
    yw = ops.linear(torch.from_numpy(xp).to(DEV), [], [], [], [], [], 0, w, ends, [cb, cb], [300, 128])
    assert yw.shape == (6, 428)
    assert torch.count_nonzero(yw[:, 256:300]) == 0
    full = ops.linear(torch.from_numpy(xp).to(DEV), [], [], [], [], [], 0, w, ends, [cb, cb], ns)
    assert torch.equal(yw[:, :256], full[:, :256]) and torch.equal(yw[:, 300:], full[:, 256:])
