"""Generates tests/golden/exl3_golden.npz by running the reference's own Python decoder.

    python tests/golden/make_golden.py --reference-src <checkout of 0xSero/trellis-serve>/core/src

The reference (`trellis_core.reference`, core/src/trellis_core/reference.py) is imported in place, never
copied.  The fixture pins the oracle and, through it, the CUDA kernels:

* codebook tables: sha256 of all 65536 fp16 values per codebook, the values at the known-answer states of
  core/tests/test_reference.py:21 and at 64 further states;
* decode: for K = 2..8 x 3 codebooks, a small ragged trellis (2 x 3 tiles) with its full decoded weight, and
  the sha256 of the decoded weight of a 128 x 256 matrix whose trellis is regenerated from the seed;
* states: decode_states of one tile per K;
* forward: linear_forward and weight_orig on (k, n) = (256, 128) for a few (K, codebook), 4 rows;
* Hadamard: had_rows on a seeded (3, 256) input.

Inputs come from numpy's PCG64 (`default_rng(seed)`), so they can be regenerated anywhere.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np


def seeded_trellis(seed: int, kt: int, nt: int, K: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.integers(0, 65536, size=(kt, nt, 16 * K), dtype=np.uint16)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-src", required=True, help="path of the reference's core/src directory")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "exl3_golden.npz"))
    args = ap.parse_args()
    sys.path.insert(0, args.reference_src)
    import torch
    from trellis_core import reference as ref

    out: dict[str, np.ndarray] = {}
    known = np.array([0, 1, 0xB38D, 0x7FFF, 0xFFFF, 12345], dtype=np.int64)
    extra = np.random.default_rng(7).integers(0, 65536, size=64)
    probe = np.concatenate([known, extra])
    out["lut_probe_states"] = probe
    for cb in (0, 1, 2):
        lut = ref.codebook_lut(cb).numpy()
        out[f"lut_sha_cb{cb}"] = np.array(sha(lut.view(np.uint16)))
        out[f"lut_probe_cb{cb}"] = lut.view(np.uint16)[probe]
        out[f"lut_moments_cb{cb}"] = np.array([lut.astype(np.float64).mean(), lut.astype(np.float64).std()])

    for K in range(2, 9):
        tile = seeded_trellis(1000 + K, 1, 1, K)
        st = ref.decode_states(torch.from_numpy(tile.view(np.int16)), K).numpy().reshape(256)
        out[f"states_K{K}"] = st.astype(np.uint16)
        for cb in (0, 1, 2):
            small = seeded_trellis(2000 + 10 * K + cb, 2, 3, K)
            w = ref.reconstruct_inner(torch.from_numpy(small.view(np.int16)), K, cb).numpy()
            out[f"w_small_K{K}_cb{cb}"] = w.view(np.uint16)
            big = seeded_trellis(3000 + 10 * K + cb, 8, 16, K)
            wb = ref.reconstruct_inner(torch.from_numpy(big.view(np.int16)), K, cb).numpy()
            out[f"w_sha_K{K}_cb{cb}"] = np.array(sha(wb.view(np.uint16)))

    rng = np.random.default_rng(11)
    for K, cb in ((2, 0), (3, 0), (3, 2), (4, 1), (5, 0), (6, 1), (8, 2)):
        k, n = 256, 128
        tr = seeded_trellis(4000 + 10 * K + cb, k // 16, n // 16, K)
        suh = (rng.integers(0, 2, size=k) * 2 - 1).astype(np.float16)
        svh = (rng.standard_normal(n) * 0.1 + 1.0).astype(np.float16)
        x = rng.standard_normal((4, k)).astype(np.float16)
        tt = torch.from_numpy(tr.view(np.int16))
        y = ref.linear_forward(torch.from_numpy(x), tt, torch.from_numpy(suh), torch.from_numpy(svh), K, cb).numpy()
        wo = ref.weight_orig(tt, torch.from_numpy(suh), torch.from_numpy(svh), K, cb).numpy()
        tag = f"K{K}_cb{cb}"
        out[f"fwd_suh_{tag}"], out[f"fwd_svh_{tag}"], out[f"fwd_x_{tag}"] = suh, svh, x
        out[f"fwd_y_{tag}"] = y.astype(np.float32)
        out[f"fwd_worig_sha_{tag}"] = np.array(sha(np.round(wo.astype(np.float64), 3)))
        out[f"fwd_xw_{tag}"] = (x.astype(np.float32) @ wo.astype(np.float32)).astype(np.float32)

    hx = rng.standard_normal((3, 256)).astype(np.float32)
    out["had_x"] = hx
    out["had_y"] = ref.had_rows(torch.from_numpy(hx)).numpy()

    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    main()
