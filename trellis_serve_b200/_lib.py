"""ctypes binding of libexl3_b200.so, the C-ABI library of sm_100a kernels (include/exl3_b200.h).

There is no fallback: if the library is missing or a call fails, an exception says so.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libexl3_b200.so")

F16, BF16, F32 = 0, 1, 2
CB_3INST, CB_MCG, CB_MUL1 = 0, 1, 2

_lib = None
_initialised: set[int] = set()

_vp, _i, _sz, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_int64
_ip = ctypes.POINTER(ctypes.c_int)

# name -> (restype, argtypes); mirrors include/exl3_b200.h one to one
SIGNATURES = {
    "exl3_status_str": (ctypes.c_char_p, [_i]),
    "exl3_last_cuda_error": (_i, []),
    "exl3_version": (_i, []),
    "exl3_init_device": (_i, [_i]),
    "exl3_device_sm_count": (_i, [_i]),
    "exl3_packed_bytes": (_sz, [_i, _i, _i]),
    "exl3_repack": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "exl3_unpack": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "exl3_reconstruct": (_i, [_vp, _i, _i, _i, _i, _vp, _vp]),
    "exl3_reconstruct_packed": (_i, [_vp, _i, _i, _i, _i, _vp, _vp]),
    "exl3_had_in": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _vp]),
    "exl3_had_out": (_i, [_vp, _i, _vp, _i, _i, _vp, _i64, _i, _vp]),
    "exl3_linear_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "exl3_linear": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _ip, _i, _i, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "exl3_rotate_fragments": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    "exl3_rmsnorm_rotate": (_i, [_vp, _vp, _vp, ctypes.c_float, _i, _vp, _i, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "exl3_silu_mul_rotate": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "exl3_linear_prerotated": (_i, [_vp, _i, _i, _vp, _ip, _i, _i, _i, _i, _vp, _i, _vp, _sz, ctypes.POINTER(_vp), _i, _i, _sz, _vp, _vp, _vp, _vp,
                                    _vp]),
    "exl3_rmsnorm_linear": (_i, [_vp, _i, _vp, _vp, _vp, ctypes.c_float, _vp, _i, _i, _vp, _vp, _ip, _i, _i, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "exl3_residual_ssq": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "exl3_normed_linear": (_i, [_vp, _i, _vp, _vp, ctypes.c_float, _vp, _i, _i, _vp, _vp, _ip, _i, _i, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "exl3_glu_linear": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _ip, _i, _i, _i, _i, _vp, _i, _vp, _sz, ctypes.POINTER(_vp), _i, _i, _sz, _vp, _vp, _vp, _vp,
                             _vp]),
    "exl3_attention_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "exl3_rope_append": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp]),
    "exl3_decode_attention": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, ctypes.c_float, _vp, _sz, _vp, _vp, _i, _vp, _sz, _vp]),
    "exl3_rope_decode_attention": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, ctypes.c_float, _vp, _sz, _vp, _vp, _i, _vp, _sz,
                                        _vp]),
    "exl3_gemm_tc_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "exl3_linear_tc": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _ip, _i, _i, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "exl3_linear_static": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _ip, _i, _i, _i, _i, _vp, _i, _vp]),
    "exl3_static_workspace_bytes": (_sz, []),
    "exl3_gemm_rotated": (_i, [_vp, _vp, _i, _i, _ip, _i, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "exl3_gemm_rotated_f32": (_i, [_vp, _vp, _i, _i, _ip, _i, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "exl3_allreduce_region_bytes": (_sz, [_sz]),
    "exl3_allreduce": (_i, [_vp, _i, _sz, ctypes.POINTER(_vp), _i, _i, _sz, _vp, _vp]),
    "exl3_linear_allreduce": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _ip, _i, _i, _i, _i, _vp, _i, _vp, _sz, ctypes.POINTER(_vp), _i, _i, _sz, _vp, _vp]),
    "exl3_moe_block_rows": (_i, []),
    "exl3_moe_sorted_capacity": (_sz, [_i, _i]),
    "exl3_moe_align": (_i, [_vp, _i, _i, _vp, _i, _vp, _vp, _vp]),
    "exl3_moe_align_mapped": (_i, [_vp, _i, _i, _vp, _i, _vp, _i, _vp, _vp, _vp]),
    "exl3_moe_fragment_bytes": (_sz, [_i, _i, _i, _i]),
    "exl3_moe_had_in": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _vp]),
    "exl3_moe_glu_had_in": (_i, [_vp, _vp, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _vp]),
    "exl3_moe_workspace_bytes": (_sz, [_i, _i]),
    "exl3_moe_gemm": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "exl3_moe_combine": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp]),
    "exl3_moe_tc_block_rows": (_i, []),
    "exl3_moe_tc_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "exl3_moe_tc_experts": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp]),
    "exl3_device_error": (_i, [_vp, _sz, _vp]),
    "exl3_set_gemv_mode": (None, [_i]),
    "exl3_set_tc_tiling": (None, [_i]),
    "exl3_set_tc_ksplit": (None, [_i]),
}


class Exl3Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, where: str, message: str):
        super().__init__(f"{where}: {message} (status {status})")
        self.status = status


def load() -> ctypes.CDLL:
    """The shared library; raises if it has not been built (python -m trellis_serve_b200.csrc.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m trellis_serve_b200.csrc.build` "
                              f"(needs nvcc); there is no fallback implementation")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        lib = load()
        msg = lib.exl3_status_str(status).decode()
        if status == 6:
            msg += f" (cudaError {lib.exl3_last_cuda_error()})"
        raise Exl3Error(status, where, msg)


def init_device(index: int) -> None:
    """Per-device set-up; must precede any CUDA-graph capture."""
    if index not in _initialised:
        check(load().exl3_init_device(index), "exl3_init_device")
        _initialised.add(index)


def sm_count(index: int) -> int:
    """Multiprocessors of device `index` as recorded at initialisation."""
    init_device(index)
    return int(load().exl3_device_sm_count(index))


def int_array(values):
    values = list(values)
    return (ctypes.c_int * max(len(values), 1))(*values) if values else None
