"""GPU parity of the dense EXL3 linear, through the C ABI, against the CPU oracle.

Tier 1 (bit-exact): decoded weights from both layouts, and weights read out through the GEMV with identity rows
(one-hot inputs make every fp32 accumulator an exact copy of one weight: the level-1 design of the reference's
cuda/src/sglang_exl3/parity/marlin_parity.py:149-183 and xpu/tests/test_bitexact_xpu.py:60-95).
Tier 2 (numerical): forward against the oracle's fp32 forward, max|d|/rms(ref) <= 2e-3 and relative L2 <= 2e-3
(marlin_parity.py:193-195, xpu/tests/oracle_cuda.py:59-64).
Plus the operator promises: determinism, CUDA-graph replay, zeros, bf16 boundary, fused groups, rows == 0.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200 import layout
from trellis_serve_b200.kernels import linear as lin

pytestmark = pytest.mark.gpu
TOL = 2e-3
DEV = "cuda:0"


def _t(a: np.ndarray) -> torch.Tensor:
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _case(seed, k, n, K, rows, sign_only=True):
    rng = np.random.default_rng(seed)
    tr = seeded_trellis(seed, k // 16, n // 16, K)
    if sign_only:
        suh, svh = seeded_signs(seed + 1, k), seeded_signs(seed + 2, n)
    else:
        suh = (rng.standard_normal(k) * 0.1 + 1.0).astype(np.float16)
        svh = (rng.standard_normal(n) * 0.1 + 1.0).astype(np.float16)
    x = rng.standard_normal((rows, k)).astype(np.float16)
    return tr, suh, svh, x


# ------------------------------------------------------------------------------------------------ tier 1

@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("K", range(2, 9))
def test_reconstruct_from_the_stored_stream_is_bit_exact(golden, K, cb):
    small = seeded_trellis(2000 + 10 * K + cb, 2, 3, K)                   # ragged: 2 x 3 tiles (fixture inputs)
    w = lin.reconstruct(_t(small), cb)
    assert np.array_equal(_bits16(w), golden[f"w_small_K{K}_cb{cb}"])
    big = seeded_trellis(3000 + 10 * K + cb, 8, 16, K)
    w = lin.reconstruct(_t(big), cb)
    assert np.array_equal(_bits16(w), orc.c_reconstruct(big, K, cb).view(np.uint16))


@pytest.mark.parametrize("K", range(2, 9))
def test_repack_matches_the_host_model_and_inverts(K):
    tr = seeded_trellis(60 + K, 16, 24, K)
    packed = lin.prepare_matrix(_t(tr))
    assert packed.numel() * 4 == tr.nbytes                                # same bytes: a permutation
    assert np.array_equal(packed.cpu().numpy().view(np.uint32), layout.repack(tr, K))
    assert np.array_equal(_bits16(lin.unprepare_matrix(packed)), tr)


@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("K", range(2, 9))
def test_reconstruct_from_the_resident_layout_is_bit_exact(K, cb):
    tr = seeded_trellis(90 + 10 * K + cb, 24, 16, K)                      # k = 384, n = 256
    w = lin.reconstruct_packed(lin.prepare_matrix(_t(tr)), cb)
    assert np.array_equal(_bits16(w), orc.c_reconstruct(tr, K, cb).view(np.uint16))


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("K", range(2, 9))
def test_identity_rows_read_the_decoded_weights_out_exactly(K, cb, mode):
    k, n = 256, 256
    tr = seeded_trellis(300 + 10 * K + cb, k // 16, n // 16, K)
    want = orc.c_reconstruct(tr, K, cb).view(np.uint16)
    packed = lin.prepare_matrix(_t(tr))
    lin.set_gemv_mode(mode)
    try:
        eye = torch.eye(k, dtype=torch.float16, device=DEV)
        got = lin.gemm_rotated(eye, packed, cb)                           # 256 rows, 16 per launch
    finally:
        lin.set_gemv_mode(-1)
    assert np.array_equal(_bits16(got), want)


def test_full_size_decode_checksum_against_the_oracle():
    """The 4096 x 4096, K = 4, 3INST configuration: every decoded weight equal to the oracle's."""
    K, cb = 4, 0
    tr = seeded_trellis(0, 256, 256, K)
    want = orc.c_reconstruct(tr, K, cb).view(np.uint16)
    t = _t(tr)
    assert np.array_equal(_bits16(lin.reconstruct(t, cb)), want)
    assert np.array_equal(_bits16(lin.reconstruct_packed(lin.prepare_matrix(t), cb)), want)


# ------------------------------------------------------------------------------------------------ tier 2

def _forward(tr, suh, svh, x, K, cb, dtype=torch.float16):
    packed = lin.prepare_matrix(_t(tr))
    y = lin.linear(_t(x).to(dtype), packed, _t(suh), _t(svh), cb)
    torch.cuda.synchronize()
    lin.device_error(torch.device(DEV))
    return y


def _check_forward(tr, suh, svh, x, K, cb):
    """The accuracy bound is measured on the fp32 accumulators (y_dtype fp32); the fp16 result the operator returns
    must be exactly those values rounded once, so its own error is the bound plus half an fp16 ulp of each output."""
    packed, xs, s, v = lin.prepare_matrix(_t(tr)), _t(x), _t(suh), _t(svh)
    y32 = torch.empty((x.shape[0], tr.shape[1] * 16), dtype=torch.float32, device=DEV)
    lin.linear(xs, packed, s, v, cb, out=y32)
    y16 = lin.linear(xs, packed, s, v, cb)
    torch.cuda.synchronize()
    lin.device_error(torch.device(DEV))
    ref = orc.c_linear_forward(x, tr, suh, svh, K, cb)
    y32n = y32.cpu().numpy()
    assert orc.max_over_rms(y32n, ref) <= TOL, orc.max_over_rms(y32n, ref)
    assert orc.rel_norm(y32n, ref) <= TOL
    assert torch.equal(y16, y32.to(torch.float16))
    assert orc.rel_norm(y16.float().cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("K,cb", [(2, 0), (3, 0), (3, 1), (3, 2), (4, 0), (4, 1), (5, 2), (6, 1), (7, 0), (8, 2)])
@pytest.mark.parametrize("rows", [1, 2, 3, 8, 9, 16])
def test_forward_matches_the_oracle(K, cb, rows, mode):
    k, n = 512, 384
    tr, suh, svh, x = _case(500 + 10 * K + cb + rows, k, n, K, rows, sign_only=False)
    lin.set_gemv_mode(mode)
    try:
        _check_forward(tr, suh, svh, x, K, cb)
    finally:
        lin.set_gemv_mode(-1)


@pytest.mark.parametrize("k,n,K,rows", [(2048, 2560, 3, 1), (2048, 2560, 3, 4), (5120, 1024, 3, 1), (1024, 5120, 4, 16),
                                        (4096, 4096, 4, 1), (640, 5120, 3, 1), (2176, 640, 5, 2), (128, 128, 3, 1)])
def test_forward_on_layer_shapes(k, n, K, rows):
    """Shapes where a CTA streams several units, crosses column-block boundaries and shares blocks with others;
    includes the tensor-parallel shard shapes of the 27B layers (640, 2176 wide)."""
    tr, suh, svh, x = _case(700 + k + n, k, n, K, rows)
    _check_forward(tr, suh, svh, x, K, 0)


@pytest.mark.parametrize("rows", [17, 40, 64])
def test_more_than_sixteen_rows_are_processed_in_chunks(rows):
    K, cb, k, n = 4, 1, 512, 256
    tr, suh, svh, x = _case(800 + rows, k, n, K, rows)
    _check_forward(tr, suh, svh, x, K, cb)


def test_fused_group_equals_its_matrices():
    """q/k/v-style group: one launch, three matrices with their own suh, adjacent output spans (layout.py:1-8)."""
    K, cb, k, rows = 3, 0, 1024, 2
    ns = [512, 128, 256]
    parts = [_case(900 + i, k, n, K, rows) for i, n in enumerate(ns)]
    x = parts[0][3]
    trs, suhs, svhs = [_t(p[0]) for p in parts], [_t(p[1]) for p in parts], [_t(p[2]) for p in parts]
    ok, why = lin.supports(trs, ns, [cb] * 3)
    assert ok, why
    b, suh_cat, svh_cat, ends = lin.prepare(trs, suhs, svhs)
    assert ends == [512, 640]
    y = lin.run(_t(x), b, suh_cat, svh_cat, ends, cb).float().cpu().numpy()
    col = 0
    for (tr, suh, svh, _), n in zip(parts, ns):
        ref = orc.c_linear_forward(x, tr, suh, svh, K, cb)
        assert orc.rel_norm(y[:, col:col + n], ref) <= TOL
        single = lin.linear(_t(x), lin.prepare_matrix(_t(tr)), _t(suh), _t(svh), cb)
        assert torch.equal(single.cpu(), torch.from_numpy(y[:, col:col + n]).half())     # same bits as a lone launch
        col += n


@pytest.mark.parametrize("rows,dtype", [(1, torch.float16), (2, torch.bfloat16), (5, torch.float16), (16, torch.bfloat16)])
def test_output_transform_inside_the_launch_equals_a_launch_of_its_own(rows, dtype):
    """exl3_linear (rotations fused into the GEMV where the row count allows) == exl3_had_in -> exl3_gemm_rotated_f32 ->
    exl3_had_out, bit for bit, fp16 and bf16 (the reference's check_inlaunch, cuda/src/sglang_exl3/parity/marlin_parity.py:114-127)."""
    K, cb, k, ns = 3, 0, 1024, [640, 384]
    parts = [_case(1400 + i, k, n, K, rows, sign_only=False) for i, n in enumerate(ns)]
    x = _t(parts[0][3]).to(dtype)
    b, suh_cat, svh_cat, ends = lin.prepare([_t(p[0]) for p in parts], [_t(p[1]) for p in parts], [_t(p[2]) for p in parts])
    fused = lin.run(x, b, suh_cat, svh_cat, ends, cb)
    xh = lin.had_in_group(x, suh_cat)
    rot = lin.gemm_rotated_group(xh, b, ends, cb, out=torch.empty((rows, sum(ns)), dtype=torch.float32, device=DEV))
    apart = torch.empty((rows, sum(ns)), dtype=dtype, device=DEV)
    col = 0
    for n in ns:
        lin.had_out_into(rot[:, col:col + n].contiguous(), svh_cat[col:col + n], apart, col)
        col += n
    torch.cuda.synchronize()
    assert torch.equal(fused.view(torch.int16), apart.view(torch.int16))


# ------------------------------------------------------------------------------------------------ promises

def test_results_are_deterministic_and_survive_graph_replay():
    K, cb, k, n, rows = 3, 0, 2048, 1280, 4
    tr, suh, svh, x = _case(1000, k, n, K, rows)
    packed, s, v = lin.prepare_matrix(_t(tr)), _t(suh), _t(svh)
    xs = _t(x)
    first = lin.linear(xs, packed, s, v, cb).clone()
    for _ in range(20):
        assert torch.equal(lin.linear(xs, packed, s, v, cb), first)
    out = torch.empty_like(first)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        lin.linear(xs, packed, s, v, cb, out=out)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        lin.linear(xs, packed, s, v, cb, out=out)
    x2 = _t(np.random.default_rng(5).standard_normal((rows, k)).astype(np.float16))
    eager = lin.linear(x2, packed, s, v, cb).clone()
    xs.copy_(x2)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)


def test_zero_input_gives_exact_zeros_and_rows_zero_is_a_noop():
    K, cb, k, n = 4, 0, 512, 256
    tr, suh, svh, _ = _case(1100, k, n, K, 1)
    packed = lin.prepare_matrix(_t(tr))
    y = lin.linear(torch.zeros((3, k), dtype=torch.float16, device=DEV), packed, _t(suh), _t(svh), cb)
    assert torch.count_nonzero(y) == 0
    y0 = lin.linear(torch.zeros((0, k), dtype=torch.float16, device=DEV), packed, _t(suh), _t(svh), cb)
    assert y0.shape == (0, n)


def test_bf16_boundary_equals_explicit_casts():
    """run(x_bf16) == run(x_bf16.half()).bfloat16() bit for bit, out-of-range magnitudes included (marlin.py:9-12)."""
    K, cb, k, n, rows = 4, 1, 512, 256, 4
    tr, suh, svh, x = _case(1200, k, n, K, rows)
    packed, s, v = lin.prepare_matrix(_t(tr)), _t(suh), _t(svh)
    xb = _t(x).to(torch.bfloat16)
    xb[0, 5] = 3.0e38
    xb[1, 7] = -1.0e5
    got = lin.linear(xb, packed, s, v, cb)
    want = lin.linear(xb.to(torch.float16), packed, s, v, cb).to(torch.bfloat16)
    assert got.dtype == torch.bfloat16
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_adversarial_inputs_stay_finite_and_accurate():
    """Large magnitudes (outputs near 1e4, inside fp16 range), small ones, and activations in the fp16 denormal
    range.  The rotated activations are fp16 (as in the reference's kernels, cuda/csrc/exl3_had.cuh:60-62), so inputs
    that land in the denormal range keep only a few significant bits: there the result must stay finite and close
    in norm, not meet the 2e-3 bound."""
    K, cb, k, n = 4, 0, 512, 256
    tr, suh, svh, _ = _case(1300, k, n, K, 1)
    rng = np.random.default_rng(3)
    big = (rng.standard_normal((2, k)) * 300.0).astype(np.float16)
    small = (rng.standard_normal((2, k)) * 1e-2).astype(np.float16)
    for x in (big, small):
        _check_forward(tr, suh, svh, x, K, cb)
    tiny = (rng.standard_normal((2, k)) * 3e-6).astype(np.float16)
    y = _forward(tr, suh, svh, tiny, K, cb).float().cpu().numpy()
    ref = orc.c_linear_forward(tiny, tr, suh, svh, K, cb)
    assert np.isfinite(y).all()
    assert orc.rel_norm(y, ref) <= 5e-2


def test_had_in_and_had_out_building_blocks():
    k, n, rows = 384, 256, 5
    rng = np.random.default_rng(9)
    x = rng.standard_normal((rows, k)).astype(np.float16)
    suh = np.stack([seeded_signs(1, k), (rng.standard_normal(k) * 0.2 + 1).astype(np.float16)])
    xh = lin.had_in_group(_t(x), _t(suh)).float().cpu().numpy()
    for s in range(2):
        ref = orc.c_had_rows(x.astype(np.float32) * suh[s].astype(np.float32))
        assert np.abs(xh[s * rows:(s + 1) * rows] - ref).max() <= 2e-3 * np.abs(ref).max()
    y = rng.standard_normal((rows, n)).astype(np.float32)
    svh = (rng.standard_normal(n) * 0.2 + 1).astype(np.float16)
    out = torch.zeros((rows, n + 128), dtype=torch.bfloat16, device=DEV)
    lin.had_out_into(_t(y), _t(svh), out, 128)
    ref = orc.c_had_rows(y) * svh.astype(np.float32)
    got = out[:, 128:].float().cpu().numpy()
    assert np.abs(got - ref).max() <= 1e-2 * np.abs(ref).max()           # bf16 output
    assert torch.count_nonzero(out[:, :128]) == 0


def test_unsupported_requests_raise():
    with pytest.raises(RuntimeError):
        lin.prepare_matrix(torch.zeros((4, 8, 48), dtype=torch.int16, device=DEV))       # k = 64
    with pytest.raises(RuntimeError):
        lin.prepare_matrix(torch.zeros((8, 8, 48), dtype=torch.int16))                   # CPU tensor: no fallback
    ok, why = lin.supports([torch.zeros((8, 8, 24), dtype=torch.int16)], [128], [0])
    assert not ok and "K" in why


@pytest.mark.parametrize("rows", [1, 4, 9])
def test_one_workspace_serves_calls_of_any_shape_in_any_order(rows):
    """The workspace is shared by every call on a device.  The split-k counters must read zero at the start of each launch
    whatever ran before: a wide matrix after a narrow one (whose scratch once lay where the wide one's counters are),
    and back, gives the bits of the same call on a fresh workspace."""
    dev = torch.device(DEV)
    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    from trellis_serve_b200.runtime.layerset import random_packed, random_signs

    def make(k, n):
        return random_packed(k, n, 3, gen, dev), random_signs(k, gen, dev, 1), (random_signs(n, gen, dev).view(-1) / 16).half()
    narrow, wide = make(2048, 1024), make(1024, 34816)
    xn = torch.randn((rows, 2048), device=dev, generator=gen).half()
    xw = torch.randn((rows, 1024), device=dev, generator=gen).half()
    lin._workspace.clear()
    fresh_wide = lin.run(xw, *wide, [], 0).clone()
    lin._workspace.clear()
    fresh_narrow = lin.run(xn, *narrow, [], 0).clone()
    for _ in range(2):
        assert torch.equal(lin.run(xw, *wide, [], 0), fresh_wide)
        assert torch.equal(lin.run(xn, *narrow, [], 0), fresh_narrow)
    lin.device_error(dev)
