"""EXL3 tensor-level rules: what the tensors stored under one quantized linear must look like.

Everything is derived from tensor names, dtypes and shapes found in safetensors headers.  Same public names and
error messages as the reference's format layer (core/src/trellis_core/format/spec.py of 0xSero/trellis-serve),
so loaders written against it keep working:

  trellis  int16 [k/16, n/16, 16K]     one 16x16 tile per (i, j), 256*K bits per tile
  suh/svh  fp16  [k] / [n]             input / output sign-scale vectors (legacy: su/sv int16 sign bit fields)
  mcg|mul1 int32 scalar                codebook marker; neither means 3INST
  bias     fp16|fp32 [n]               optional

k and n are the stored widths, padded to the 128-wide Hadamard block.  K may be 1..8, or 1.5 / 2.5 / 3.5 with
the mul1 codebook (spec.py:41-68 of the reference).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Mapping

BLOCK = 128
TILE = 16
MCG_MULTIPLIER = 0xCBAC1FED
MUL1_MULTIPLIER = 0x83DCD12D

REQUIRED_TRELLIS = "trellis"
INPUT_SCALE = ("suh", "su")
OUTPUT_SCALE = ("svh", "sv")
MARKERS = ("mcg", "mul1")
KNOWN_SUFFIXES = frozenset((REQUIRED_TRELLIS,) + INPUT_SCALE + OUTPUT_SCALE + MARKERS + ("bias",))


class FormatError(ValueError):
    """The checkpoint does not have the EXL3 structure this code can run."""


class Codebook(enum.Enum):
    INST3 = "3inst"
    MCG = "mcg"
    MUL1 = "mul1"

    @property
    def kernel_id(self) -> int:
        """Codebook number the kernels take (0 3inst, 1 mcg, 2 mul1)."""
        return {"3inst": 0, "mcg": 1, "mul1": 2}[self.value]


@dataclass(frozen=True, order=True)
class BitsK:
    """Bits per weight, stored doubled so the half-integer rates stay exact."""
    twice: int

    @property
    def value(self) -> float:
        return self.twice / 2

    @property
    def is_half(self) -> bool:
        return bool(self.twice & 1)

    @property
    def trellis_words(self) -> int:
        return 8 * self.twice

    @classmethod
    def from_trellis_words(cls, words: int, codebook: Codebook) -> "BitsK":
        twice, rem = divmod(words, 8)
        if rem or twice < 2 or twice > 16:
            raise FormatError(f"trellis last dim {words} is not a valid EXL3 bitrate")
        bits = cls(twice)
        if bits.is_half:
            if twice not in (3, 5, 7):
                raise FormatError(f"half-integer K={bits.value} is not defined (only 1.5, 2.5, 3.5)")
            if codebook is not Codebook.MUL1:
                raise FormatError(f"half-integer K={bits.value} requires the mul1 codebook, got {codebook.value}")
        return bits

    def __str__(self) -> str:
        return f"{self.value:g}"


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple[int, ...]
    file: str = ""
    nbytes: int = 0


@dataclass(frozen=True)
class MatrixSpec:
    """One stored EXL3 linear: y = Had(x * suh) @ W -> Had -> * svh (+ bias); the trellis is (k/16, n/16, words),
    input dimension first."""
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
        return sum(t.nbytes for t in self.tensors.values())

    def same_kernel_class(self, other: "MatrixSpec") -> bool:
        return (self.k, self.n, self.bits, self.codebook) == (other.k, other.n, other.bits, other.codebook)


def _pick_one(tensors: Mapping[str, TensorInfo], names: tuple[str, str], key: str) -> tuple[str, TensorInfo]:
    found = [n for n in names if n in tensors]
    if len(found) != 1:
        raise FormatError(f"{key}: expected exactly one of {names}, found {found or 'none'}")
    return found[0], tensors[found[0]]


def build_matrix_spec(key: str, tensors: Mapping[str, TensorInfo]) -> MatrixSpec:
    """Validate everything stored as `<key>.<suffix>` and describe the linear.  Refuses, with a reason, anything
    that is not stock EXL3 rather than guessing."""
    extra = sorted(set(tensors) - KNOWN_SUFFIXES)
    if extra:
        raise FormatError(f"{key}: unknown tensors {extra} under an EXL3 linear (derivative or newer format; refusing to guess)")
    tr = tensors.get(REQUIRED_TRELLIS)
    if tr is None:
        raise FormatError(f"{key}: no .trellis tensor")
    if tr.dtype != "I16" or len(tr.shape) != 3:
        raise FormatError(f"{key}.trellis: expected 3-D I16, got {tr.dtype} {tr.shape}")
    present = [m for m in MARKERS if m in tensors]
    if len(present) == 2:
        raise FormatError(f"{key}: both .mcg and .mul1 markers present")
    for m in present:
        t = tensors[m]
        if t.dtype != "I32" or t.shape not in ((), (1,)):
            raise FormatError(f"{key}.{m}: expected I32 scalar, got {t.dtype} {t.shape}")
    codebook = Codebook(present[0]) if present else Codebook.INST3
    k, n = tr.shape[0] * TILE, tr.shape[1] * TILE
    if k % BLOCK or n % BLOCK:
        raise FormatError(f"{key}: stored dims ({k}, {n}) are not multiples of {BLOCK}")
    bits = BitsK.from_trellis_words(tr.shape[2], codebook)
    in_name, in_t = _pick_one(tensors, INPUT_SCALE, key)
    out_name, out_t = _pick_one(tensors, OUTPUT_SCALE, key)
    legacy = in_name == "su" or out_name == "sv"
    if legacy and (in_name, out_name) != ("su", "sv"):
        raise FormatError(f"{key}: mixed legacy/modern scale tensors ({in_name}, {out_name})")
    dtype, in_shape, out_shape = ("I16", (k // TILE,), (n // TILE,)) if legacy else ("F16", (k,), (n,))
    for t, shape in ((in_t, in_shape), (out_t, out_shape)):
        if t.dtype != dtype or t.shape != shape:
            raise FormatError(f"{t.name}: expected {dtype} {shape}, got {t.dtype} {t.shape}")
    bias = tensors.get("bias")
    if bias is not None and (bias.dtype not in ("F16", "F32") or bias.shape != (n,)):
        raise FormatError(f"{key}.bias: expected F16/F32 ({n},), got {bias.dtype} {bias.shape}")
    return MatrixSpec(key, k, n, bits, codebook, bias is not None, legacy, dict(tensors))
