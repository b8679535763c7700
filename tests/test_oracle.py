"""Pins the CPU oracle (oracle/) against the reference decoder's own outputs (tests/golden/exl3_golden.npz,
made by tests/golden/make_golden.py from core/src/trellis_core/reference.py) and against the known-answer
material of the reference's core/tests/test_reference.py."""
from __future__ import annotations

import hashlib
import struct

import numpy as np
import pytest

from conftest import seeded_trellis
from oracle import exl3_oracle as orc


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _mcg_scalar(state: int) -> float:
    """MCG value of one state written out independently (same check as core/tests/test_reference.py:10-22)."""
    x = (state * 0xCBAC1FED) & 0xFFFFFFFF
    x = ((x & 0x8FFF8FFF) ^ 0x3B603B60) & 0xFFFFFFFF
    lo = np.frombuffer(struct.pack("<H", x & 0xFFFF), dtype=np.float16)[0]
    hi = np.frombuffer(struct.pack("<H", x >> 16), dtype=np.float16)[0]
    return float(np.float16(np.float64(lo) + np.float64(hi)))


@pytest.mark.parametrize("impl", ["np", "c"])
def test_mcg_known_answer_states(impl):
    lut = (orc.np_codebook_lut if impl == "np" else orc.c_codebook_lut)(orc.CB_MCG).astype(np.float32)
    for s in (0, 1, 0xB38D, 0x7FFF, 0xFFFF, 12345):
        assert lut[s] == _mcg_scalar(s), hex(s)


@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("impl", ["np", "c"])
def test_codebook_tables_match_the_reference(golden, impl, cb):
    lut = (orc.np_codebook_lut if impl == "np" else orc.c_codebook_lut)(cb)
    assert lut.shape == (65536,)
    assert _sha(lut.view(np.uint16)) == str(golden[f"lut_sha_cb{cb}"])
    probe = golden["lut_probe_states"]
    assert np.array_equal(lut.view(np.uint16)[probe], golden[f"lut_probe_cb{cb}"])
    v = lut.astype(np.float64)
    assert abs(v.mean()) < 0.05 and 1.0 < v.std() < 1.5          # core/tests/test_reference.py:26-30
    assert np.allclose([v.mean(), v.std()], golden[f"lut_moments_cb{cb}"])


@pytest.mark.parametrize("K", range(2, 9))
def test_states_match_the_reference(golden, K):
    tile = seeded_trellis(1000 + K, 1, 1, K)
    want = golden[f"states_K{K}"]
    assert np.array_equal(orc.np_decode_states(tile, K).reshape(256), want)
    assert np.array_equal(orc.c_decode_states(tile.reshape(-1), K), want)


@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("K", range(2, 9))
def test_decoded_weights_match_the_reference_bit_for_bit(golden, K, cb):
    small = seeded_trellis(2000 + 10 * K + cb, 2, 3, K)                      # ragged: 2 x 3 tiles
    want = golden[f"w_small_K{K}_cb{cb}"]
    assert np.array_equal(orc.np_reconstruct(small, K, cb).view(np.uint16), want)
    assert np.array_equal(orc.c_reconstruct(small, K, cb).view(np.uint16), want)
    big = seeded_trellis(3000 + 10 * K + cb, 8, 16, K)
    sha = str(golden[f"w_sha_K{K}_cb{cb}"])
    assert _sha(orc.np_reconstruct(big, K, cb).view(np.uint16)) == sha
    assert _sha(orc.c_reconstruct(big, K, cb).view(np.uint16)) == sha


@pytest.mark.parametrize("K,cb", [(2, 0), (3, 0), (3, 2), (4, 1), (5, 0), (6, 1), (8, 2)])
def test_forward_matches_the_reference(golden, K, cb):
    tag = f"K{K}_cb{cb}"
    tr = seeded_trellis(4000 + 10 * K + cb, 16, 8, K)
    x, suh, svh = golden[f"fwd_x_{tag}"], golden[f"fwd_suh_{tag}"], golden[f"fwd_svh_{tag}"]
    want = golden[f"fwd_y_{tag}"]
    for got in (orc.np_linear_forward(x, tr, suh, svh, K, cb), orc.c_linear_forward(x, tr, suh, svh, K, cb)):
        assert orc.max_over_rms(got, want) < 2e-5              # fp32 summation order only
    # forward == x @ original-basis weight (core/tests/test_reference.py:33-43; tolerance from there)
    xw = x.astype(np.float32) @ orc.np_weight_orig(tr, suh, svh, K, cb)
    assert np.allclose(xw, want, rtol=2e-2, atol=2e-2)
    assert np.allclose(xw, golden[f"fwd_xw_{tag}"], rtol=1e-3, atol=1e-3)


def test_hadamard_matches_the_reference(golden):
    x, want = golden["had_x"], golden["had_y"]
    assert np.allclose(orc.np_had_rows(x), want, atol=1e-5)
    assert np.allclose(orc.c_had_rows(x), want, atol=1e-5)
    twice = orc.c_had_rows(orc.c_had_rows(x))                  # H is symmetric and orthonormal: H H = I
    assert np.allclose(twice, x, atol=1e-5)


def test_empty_and_single_tile_inputs():
    assert orc.np_reconstruct(np.zeros((0, 4, 48), dtype=np.uint16), 3, 0).shape == (0, 64)
    assert orc.c_reconstruct(np.zeros((0, 4, 48), dtype=np.uint16), 3, 0).shape == (0, 64)
    one = seeded_trellis(5, 1, 1, 3)
    assert np.array_equal(orc.np_reconstruct(one, 3, 0).view(np.uint16), orc.c_reconstruct(one, 3, 0).view(np.uint16))


def test_all_ones_and_all_zero_streams():
    """Circular windows: a constant stream gives one state everywhere, for every K."""
    for K in range(2, 9):
        for fill, state in ((0x0000, 0x0000), (0xFFFF, 0xFFFF)):
            tile = np.full((16 * K,), fill, dtype=np.uint16)
            assert np.all(orc.c_decode_states(tile, K) == state)
            assert np.all(orc.np_decode_states(tile[None], K) == state)
