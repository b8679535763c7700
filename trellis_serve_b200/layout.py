"""Host model of the resident ("packed") trellis layout the sm_100a kernels read.

The layout is a pure permutation of the stored EXL3 bit stream (same byte count, k*n*K/8):

    packed[nb][kg][nt][kq][i][lane]  uint32
      nb   column block of 128        (n / 128)
      kg   row block of 128           (k / 128)
      nt   16-column tile in the block (8)
      kq   group of four 16-row tiles (2)
      i    word of the lane stream    (K)
      lane 32

The lane stream of (nb, kg, nt, kq, lane) is B0|B1|B2|B3 with Bt = stream bits [8K*lane, 8K*(lane+1)) of tile
(row tile kg*8 + kq*4 + t, column tile nb*8 + nt), first stream bit most significant.

`repack` / `unpack` here are the numpy twins of the device kernels (csrc/exl3_kernels.cu) and are exact inverses;
they let a loader prepare weights on the CPU and let the tests check the device kernels word for word.
`lane_states` replays, in numpy, the register-level extraction of csrc/exl3_decode.cuh (own words, one neighbour
word, byte merge, eight windows) so the bit arithmetic can be verified without a GPU.

The stored format itself is the reference's: int16 [k/16, n/16, 16K], 32-bit words from little-endian pairs,
bits MSB first (core/src/trellis_core/reference.py:10-12 of 0xSero/trellis-serve).
"""
from __future__ import annotations

import numpy as np


def _stream_bits(trellis: np.ndarray) -> np.ndarray:
    """uint16 [kt, nt, 16K] -> bits uint8 [kt, nt, 256K], stream order."""
    t16 = np.ascontiguousarray(trellis).view(np.uint16).astype(np.uint32)
    words = t16[..., 0::2] | (t16[..., 1::2] << 16)
    shifts = np.arange(31, -1, -1, dtype=np.uint32)
    return ((words[..., None] >> shifts) & 1).astype(np.uint8).reshape(*words.shape[:-1], -1)


def _bits_to_words(bits: np.ndarray) -> np.ndarray:
    """bits [..., 32m] MSB first -> uint32 [..., m]."""
    b = bits.reshape(*bits.shape[:-1], -1, 32).astype(np.uint32)
    weights = (1 << np.arange(31, -1, -1, dtype=np.uint64)).astype(np.uint32)
    return (b * weights).sum(-1, dtype=np.uint64).astype(np.uint32)


def repack(trellis: np.ndarray, K: int) -> np.ndarray:
    """Stored trellis [k/16, n/16, 16K] (k, n multiples of 128) -> packed uint32 [NB, KG, 8, 2, K, 32]."""
    kt, nt, words = trellis.shape
    if words != 16 * K or kt % 8 or nt % 8:
        raise ValueError(f"need [k/16, n/16, 16K] with k, n multiples of 128, got {trellis.shape} for K={K}")
    KG, NB = kt // 8, nt // 8
    bits = _stream_bits(trellis)                                         # [kt, nt, 256K]
    bits = bits.reshape(KG, 2, 4, NB, 8, 32, 8 * K)                      # kg, kq, t, nb, nt, lane, own bits
    bits = bits.transpose(3, 0, 4, 1, 5, 2, 6)                           # nb, kg, nt, kq, lane, t, own
    lane_stream = bits.reshape(NB, KG, 8, 2, 32, 32 * K)
    w = _bits_to_words(lane_stream)                                      # [NB, KG, 8, 2, 32, K]
    return np.ascontiguousarray(w.transpose(0, 1, 2, 3, 5, 4))           # [NB, KG, 8, 2, K, 32]


def unpack(packed: np.ndarray, K: int) -> np.ndarray:
    """Exact inverse of `repack`: packed [NB, KG, 8, 2, K, 32] -> uint16 [k/16, n/16, 16K]."""
    NB, KG = packed.shape[:2]
    w = np.ascontiguousarray(packed).reshape(NB, KG, 8, 2, K, 32).transpose(0, 1, 2, 3, 5, 4)   # ..., lane, K
    shifts = np.arange(31, -1, -1, dtype=np.uint32)
    bits = ((w[..., None] >> shifts) & 1).astype(np.uint8).reshape(NB, KG, 8, 2, 32, 4, 8 * K)  # nb,kg,nt,kq,lane,t,own
    bits = bits.transpose(1, 3, 5, 0, 2, 4, 6)                           # kg, kq, t, nb, nt, lane, own
    stream = bits.reshape(KG * 8, NB * 8, 256 * K)
    words = _bits_to_words(stream)                                       # [kt, nt, 8K]
    out = np.empty((KG * 8, NB * 8, 16 * K), dtype=np.uint16)
    out[..., 0::2] = (words & 0xFFFF).astype(np.uint16)
    out[..., 1::2] = (words >> 16).astype(np.uint16)
    return out


# ---- numpy replay of the device-side extraction (csrc/exl3_decode.cuh) ------------------------------------

def _stream_bits_ending_at(L: np.ndarray, K: int, end: int) -> np.ndarray:
    wi, r = divmod(end, 32)
    if r == 0:
        return L[..., wi - 1]
    if wi == 0:
        return L[..., 0] >> np.uint32(32 - r)
    return ((L[..., wi - 1].astype(np.uint64) << np.uint64(r)) & 0xFFFFFFFF).astype(np.uint32) | (L[..., wi] >> np.uint32(32 - r))


def _prmt(a: np.ndarray, b: np.ndarray, sel: int) -> np.ndarray:
    src = np.stack([(a >> np.uint32(8 * i)) & 0xFF for i in range(4)] + [(b >> np.uint32(8 * i)) & 0xFF for i in range(4)])
    out = np.zeros_like(a)
    for i in range(4):
        out |= src[(sel >> (4 * i)) & 0x7] << np.uint32(8 * i)
    return out


def lane_states(packed: np.ndarray, K: int, pipe_balanced: bool = False) -> np.ndarray:
    """packed [NB, KG, 8, 2, K, 32] -> states uint16 [NB, KG, 8, 2, 4 (tile), 32 (lane), 8 (element)],
    computed exactly as a warp does it: per-tile right-aligned own words, the previous lane's low word, a byte
    merge, then eight 16-bit windows.  `pipe_balanced` replays the GEMV's variant: 32-bit registers at 16-bit
    offsets of the merged bits, one multiply by a power of two and one shift right by 16 per window."""
    L = np.ascontiguousarray(packed).transpose(0, 1, 2, 3, 5, 4).astype(np.uint32)          # [..., lane, K]
    out = np.empty(L.shape[:-1][:-1] + (4, 32, 8), dtype=np.uint16)
    zero = np.zeros(L.shape[:-1], dtype=np.uint32)
    for T in range(4):
        end = 8 * K * (T + 1)
        own0 = _stream_bits_ending_at(L, K, end)
        own1 = _stream_bits_ending_at(L, K, end - 32) if 8 * K > 32 else zero
        prev0 = np.roll(own0, 1, axis=-1)                                                    # lane l gets lane l-1
        if K == 2:
            e = [_prmt(own0, prev0, 0x5410), zero, zero]
        elif K == 3:
            e = [_prmt(own0, prev0, 0x4210), prev0 >> np.uint32(8), zero]
        elif K == 4:
            e = [own0, prev0, zero]
        elif K == 5:
            e = [own0, _prmt(own1, prev0, 0x6540), zero]
        elif K == 6:
            e = [own0, _prmt(own1, prev0, 0x5410), zero]
        elif K == 7:
            e = [own0, _prmt(own1, prev0, 0x4210), prev0 >> np.uint32(8)]
        else:
            e = [own0, own1, prev0]
        if pipe_balanced:
            if K == 2:
                R = [_prmt(own0, prev0, 0x5410)]
            elif K == 3:
                R = [_prmt(own0, prev0, 0x4210), _prmt(own0, prev0, 0x6542)]
            elif K == 4:
                R = [own0, _prmt(own0, prev0, 0x5432)]
            else:
                R = [e[0], _prmt(e[0], e[1], 0x5432), e[1], _prmt(e[1], e[2], 0x5432)]
            for P in range(8):
                j, sh = divmod(K * (7 - P), 16)
                if sh == 0:
                    s = R[j] & 0xFFFF
                else:
                    s = ((R[j].astype(np.uint64) << np.uint64(16 - sh)) & 0xFFFFFFFF).astype(np.uint32) >> np.uint32(16)
                out[..., T, :, P] = s.astype(np.uint16)
            continue
        for P in range(8):
            lo = K * (7 - P)
            wi, sh = divmod(lo, 32)
            if sh + 16 <= 32:
                s = (e[wi] >> np.uint32(sh)) & 0xFFFF
            else:
                s = ((e[wi] >> np.uint32(sh)) | ((e[wi + 1].astype(np.uint64) << np.uint64(32 - sh)) & 0xFFFFFFFF).astype(np.uint32)) & 0xFFFF
            out[..., T, :, P] = s.astype(np.uint16)
    return out
