"""The tensors of one EXL3 linear and what they must look like.

A quantized linear `<key>` is stored as a handful of tensors `<key>.<suffix>`; everything needed to run it can be
read off their names, dtypes and shapes (safetensors headers), no data required:

  suffix      dtype        shape               meaning
  trellis     I16          [k/16, n/16, W]     one 16 x 16 tile of weights per (i, j); W = 16 K words = 256 K bits
  suh | su    F16 | I16    [k] | [k/16]        input signs / scales (su: one sign bit per element, legacy)
  svh | sv    F16 | I16    [n] | [n/16]        output signs / scales (sv: legacy)
  mcg, mul1   I32          scalar              codebook marker; with neither the codebook is 3INST
  bias        F16 | F32    [n]                 optional

k and n are the stored widths, multiples of the 128-element rotation block.  The bitrate K is an integer 1..8, or
1.5 / 2.5 / 3.5 with the mul1 codebook.  Public names and the wording of the errors follow
core/src/trellis_core/format/spec.py (:34-107) of 0xSero/trellis-serve, so that loaders written against it keep working.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Mapping

TILE = 16                                    # weights per tile edge
BLOCK = 128                                  # elements per rotation block
MCG_MULTIPLIER = 0xCBAC1FED
MUL1_MULTIPLIER = 0x83DCD12D

REQUIRED_TRELLIS = "trellis"
INPUT_SCALE = ("suh", "su")                  # modern, legacy
OUTPUT_SCALE = ("svh", "sv")
MARKERS = ("mcg", "mul1")
KNOWN_SUFFIXES = frozenset({REQUIRED_TRELLIS, "bias", *INPUT_SCALE, *OUTPUT_SCALE, *MARKERS})

_HALF_RATES = (3, 5, 7)                      # doubled: 1.5, 2.5, 3.5


class FormatError(ValueError):
    """The checkpoint does not have the EXL3 structure this code can run."""


class Codebook(enum.Enum):
    INST3 = "3inst"
    MCG = "mcg"
    MUL1 = "mul1"

    @property
    def kernel_id(self) -> int:
        """Number the kernels and the reference decoder use for this codebook: 0, 1, 2 in declaration order."""
        return list(Codebook).index(self)


@dataclass(frozen=True, order=True)
class BitsK:
    """A bitrate, held as twice its value so that 1.5, 2.5 and 3.5 are exact integers too."""
    twice: int

    @property
    def value(self) -> float:
        return 0.5 * self.twice

    @property
    def is_half(self) -> bool:
        return self.twice % 2 == 1

    @property
    def trellis_words(self) -> int:
        """int16 words per tile: 256 weights x K bits / 16."""
        return self.twice * (TILE * TILE) // 32

    @classmethod
    def from_trellis_words(cls, words: int, codebook: Codebook) -> "BitsK":
        if words % 8 or not 16 <= words <= 128:
            raise FormatError(f"trellis last dim {words} is not a valid EXL3 bitrate")
        rate = cls(words // 8)
        if rate.is_half and rate.twice not in _HALF_RATES:
            raise FormatError(f"half-integer K={rate.value} is not defined (only 1.5, 2.5, 3.5)")
        if rate.is_half and codebook is not Codebook.MUL1:
            raise FormatError(f"half-integer K={rate.value} requires the mul1 codebook, got {codebook.value}")
        return rate

    def __str__(self) -> str:
        return format(self.value, "g")


@dataclass(frozen=True)
class TensorInfo:
    """One header entry: where a tensor lives and how large it is."""
    name: str
    dtype: str
    shape: tuple[int, ...]
    file: str = ""
    nbytes: int = 0


@dataclass(frozen=True)
class MatrixSpec:
    """One stored EXL3 linear, y = Had(Had(x * suh) @ W) * svh (+ bias), W of shape (k, n) with the input dimension
    first."""
    key: str
    k: int
    n: int
    bits: BitsK
    codebook: Codebook
    has_bias: bool = False
    legacy_signs: bool = False
    tensors: Mapping[str, TensorInfo] = field(default_factory=dict, compare=False, repr=False)

    @property
    def nbytes(self) -> int:
        return sum(info.nbytes for info in self.tensors.values())

    def same_kernel_class(self, other: "MatrixSpec") -> bool:
        """True when one kernel configuration serves both matrices."""
        mine = (self.k, self.n, self.bits, self.codebook)
        return mine == (other.k, other.n, other.bits, other.codebook)


def _pick_one(tensors: Mapping[str, TensorInfo], names: tuple[str, str], key: str) -> tuple[str, TensorInfo]:
    present = [name for name in names if name in tensors]
    if len(present) == 1:
        return present[0], tensors[present[0]]
    raise FormatError(f"{key}: expected exactly one of {names}, found {present or 'none'}")


def _codebook_of(key: str, tensors: Mapping[str, TensorInfo]) -> Codebook:
    markers = [m for m in MARKERS if m in tensors]
    if len(markers) > 1:
        raise FormatError(f"{key}: both .mcg and .mul1 markers present")
    for m in markers:
        info = tensors[m]
        if info.dtype != "I32" or info.shape not in ((), (1,)):
            raise FormatError(f"{key}.{m}: expected I32 scalar, got {info.dtype} {info.shape}")
    return Codebook(markers[0]) if markers else Codebook.INST3


def _expect(info: TensorInfo, dtype: str, shape: tuple) -> None:
    if (info.dtype, info.shape) != (dtype, shape):
        raise FormatError(f"{info.name}: expected {dtype} {shape}, got {info.dtype} {info.shape}")


def build_matrix_spec(key: str, tensors: Mapping[str, TensorInfo]) -> MatrixSpec:
    """Checks the tensors stored under `key` (by suffix) and describes the linear.  Anything that is not stock EXL3 is
    refused with the reason instead of being guessed at."""
    unknown = sorted(set(tensors) - KNOWN_SUFFIXES)
    if unknown:
        raise FormatError(f"{key}: unknown tensors {unknown} under an EXL3 linear (derivative or newer format; refusing to guess)")
    trellis = tensors.get(REQUIRED_TRELLIS)
    if trellis is None:
        raise FormatError(f"{key}: no .trellis tensor")
    if trellis.dtype != "I16" or len(trellis.shape) != 3:
        raise FormatError(f"{key}.trellis: expected 3-D I16, got {trellis.dtype} {trellis.shape}")
    codebook = _codebook_of(key, tensors)
    k_tiles, n_tiles, words = trellis.shape
    k, n = k_tiles * TILE, n_tiles * TILE
    if k % BLOCK or n % BLOCK:
        raise FormatError(f"{key}: stored dims ({k}, {n}) are not multiples of {BLOCK}")
    bits = BitsK.from_trellis_words(words, codebook)

    in_name, in_info = _pick_one(tensors, INPUT_SCALE, key)
    out_name, out_info = _pick_one(tensors, OUTPUT_SCALE, key)
    legacy = (in_name == "su", out_name == "sv")
    if legacy[0] != legacy[1]:
        raise FormatError(f"{key}: mixed legacy/modern scale tensors ({in_name}, {out_name})")
    if legacy[0]:
        _expect(in_info, "I16", (k // TILE,))
        _expect(out_info, "I16", (n // TILE,))
    else:
        _expect(in_info, "F16", (k,))
        _expect(out_info, "F16", (n,))
    bias = tensors.get("bias")
    if bias is not None and (bias.dtype not in ("F16", "F32") or bias.shape != (n,)):
        raise FormatError(f"{key}.bias: expected F16/F32 ({n},), got {bias.dtype} {bias.shape}")
    return MatrixSpec(key=key, k=k, n=n, bits=bits, codebook=codebook, has_bias=bias is not None, legacy_signs=legacy[0],
                      tensors=dict(tensors))
