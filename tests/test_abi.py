"""The C-ABI library loads without a GPU and exports every symbol include/exl3_b200.h declares; argument
errors are reported as statuses before anything is launched."""
from __future__ import annotations

import ctypes
import os
import re

import pytest

from trellis_serve_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols() -> list[str]:
    text = open(os.path.join(ROOT, "include", "exl3_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(exl3_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = _declared_symbols()
    for must in ("exl3_init_device", "exl3_repack", "exl3_unpack", "exl3_reconstruct", "exl3_had_in", "exl3_had_out",
                 "exl3_linear", "exl3_gemm_rotated", "exl3_linear_workspace_bytes", "exl3_status_str"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/exl3_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature in trellis_serve_b200/_lib.py"


def test_status_strings_and_pure_functions():
    lib = _lib.load()
    assert lib.exl3_status_str(0) == b"ok"
    for code in range(1, 12):
        assert lib.exl3_status_str(code) not in (b"", b"unknown status")
    assert lib.exl3_status_str(999) == b"unknown status"
    assert lib.exl3_packed_bytes(4096, 4096, 4) == 8388608            # k*n*K/8: the stored size, no padding
    assert lib.exl3_packed_bytes(17408, 5120, 3) == 17408 * 5120 * 3 // 8
    assert lib.exl3_packed_bytes(128, 128, 9) == 0
    assert lib.exl3_linear_workspace_bytes(1, 5120, 5120, 1) % 256 == 0


def test_argument_errors_are_statuses_not_launches():
    """None of these reach a kernel launch, so they run on a machine without a GPU."""
    lib = _lib.load()
    nul = ctypes.c_void_p(0)
    buf = ctypes.create_string_buffer(8192)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 255) & ~255)           # 256-byte aligned, as device buffers are
    assert lib.exl3_repack(p, 100, 128, 4, p, nul) == 1                # k not a multiple of 128
    assert lib.exl3_repack(p, 128, 128, 9, p, nul) == 2                # K out of range
    assert lib.exl3_repack(nul, 128, 128, 4, p, nul) == 4              # null pointer
    assert lib.exl3_reconstruct(p, 16, 16, 1, 0, p, nul) == 2
    assert lib.exl3_reconstruct(p, 16, 16, 3, 7, p, nul) == 3          # unknown codebook
    assert lib.exl3_reconstruct(p, 0, 16, 3, 0, p, nul) == 0           # empty matrix: no-op
    assert lib.exl3_had_in(p, 2, nul, 1, 1, 128, p, nul) == 10         # fp32 activations are not accepted
    assert lib.exl3_had_in(p, 0, nul, 1, 0, 128, p, nul) == 0          # rows == 0: no-op
    assert lib.exl3_had_out(p, 0, nul, 1, 100, p, 100, 0, nul) == 1
    ends = (ctypes.c_int * 1)(64)
    assert lib.exl3_linear(p, 0, p, 3, 0, p, p, ends, 2, 1, 128, 256, p, 0, p, 4096, nul) == 1    # shard end not 128-aligned
    assert lib.exl3_linear(p, 0, p, 3, 0, p, p, None, 1, 0, 128, 256, p, 0, p, 4096, nul) == 0    # rows == 0
    assert lib.exl3_device_error(nul, 64, nul) == 5                    # (NULL, 0) names the built-in scratch instead and needs a device
    # the exchange entry points: geometry of the rank set and of the regions is checked before anything runs
    regions = (ctypes.c_void_p * 2)(p, p)
    assert lib.exl3_allreduce(p, 0, 8, regions, 2, 2, 64, p, nul) == 1                             # rank outside the world
    assert lib.exl3_allreduce(p, 0, 12, regions, 0, 2, 64, p, nul) == 1                            # n not a multiple of 8
    assert lib.exl3_allreduce(p, 2, 8, regions, 0, 2, 64, p, nul) == 10                            # fp32 is not exchanged
    assert lib.exl3_allreduce(p, 0, 8, regions, 0, 1, 64, p, nul) == 0                             # a world of one: no-op
    assert lib.exl3_linear_allreduce(p, 0, p, 3, 0, p, p, None, 1, 1, 128, 256, p, 0, p, 4096, regions, 0, 17, 64, p, nul) == 1
    assert lib.exl3_linear_allreduce(p, 0, p, 3, 0, p, p, None, 1, 1, 128, 256, p, 2, p, 4096, regions, 0, 2, 4096, p, nul) == 10
    assert lib.exl3_linear_allreduce(p, 0, p, 3, 0, p, p, None, 1, 1, 128, 256, p, 0, p, 4096, regions, 0, 2, 64, p, nul) == 1   # slot too small
    assert lib.exl3_linear_allreduce(p, 0, p, 3, 0, p, p, None, 1, 0, 128, 256, p, 0, p, 4096, regions, 0, 2, 4096, p, nul) == 0  # rows == 0
    # routing alignment of one bitrate class
    assert lib.exl3_moe_align_mapped(p, 8, 16, p, 0, p, 64, p, p, nul) == 1                        # empty class
    assert lib.exl3_moe_align_mapped(p, 8, 16, nul, 4, p, 64, p, p, nul) == 4                      # no expert map
    assert lib.exl3_moe_align_mapped(p, 8, 16, p, 4, p, 8, p, p, nul) == 1                         # sorted_ids too short


def test_missing_library_is_a_loud_error(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", os.path.join(ROOT, "no_such_dir", "libexl3_b200.so"))
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()
