"""Resident layout and register-level extraction, checked on the CPU against the oracle's states:
repack/unpack are exact inverses and the lane-local window arithmetic of csrc/exl3_decode.cuh (replayed in
numpy by trellis_serve_b200.layout.lane_states) yields the reference's states for every K."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200 import layout


@pytest.mark.parametrize("K", range(2, 9))
def test_repack_is_a_permutation_with_an_exact_inverse(K):
    tr = seeded_trellis(50 + K, 16, 24, K)                 # k = 256, n = 384
    packed = layout.repack(tr, K)
    assert packed.dtype == np.uint32 and packed.nbytes == tr.nbytes
    assert packed.shape == (3, 2, 8, 2, K, 32)
    assert np.array_equal(layout.unpack(packed, K), tr)
    # a permutation of bits keeps the population count
    assert np.unpackbits(packed.view(np.uint8)).sum() == np.unpackbits(tr.view(np.uint8)).sum()


@pytest.mark.parametrize("balanced", [False, True])
@pytest.mark.parametrize("K", range(2, 9))
def test_lane_local_extraction_gives_the_reference_states(K, balanced):
    tr = seeded_trellis(70 + K, 8, 16, K)                  # k = 128, n = 256
    packed = layout.repack(tr, K)
    got = layout.lane_states(packed, K, balanced)                    # [NB, KG, 8 nt, 2 kq, 4 t, 32 lane, 8]
    want = orc.np_decode_states(tr, K)                     # [kt, nt, 256]
    NB, KG = packed.shape[:2]
    for nb in range(NB):
        for kg in range(KG):
            for nt in range(8):
                for kq in range(2):
                    for t in range(4):
                        ref = want[kg * 8 + kq * 4 + t, nb * 8 + nt].reshape(32, 8)
                        assert np.array_equal(got[nb, kg, nt, kq, t], ref), (K, nb, kg, nt, kq, t)


def test_repack_rejects_shapes_that_are_not_128_multiples():
    with pytest.raises(ValueError):
        layout.repack(np.zeros((4, 8, 48), dtype=np.uint16), 3)
    with pytest.raises(ValueError):
        layout.repack(np.zeros((8, 8, 48), dtype=np.uint16), 4)
