"""exl3_linear_static: the fused linear whose scratch is a fixed array inside the library.

Some hosts of this library cannot allocate device memory at the point where they call a linear: a plugin hook that
is handed nothing but the tensors of the call, code running inside a region of another framework where its caching
allocator must not be touched, or an embedder that gives out all device memory once at start-up.  For them the
library carries its own scratch.  This test calls that entry point directly through the C ABI, twice in a row
(the second call meets whatever the first left in the shared array), and requires the same bits as exl3_linear
with a caller-owned workspace.  It lives in a file pytest collects last, and passes on its own in a fresh process
as well as after the other tests.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from conftest import seeded_signs, seeded_trellis
from trellis_serve_b200 import _lib
from trellis_serve_b200.kernels import linear as lin

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _static_linear(x, packed, suh, svh, ends, K, cb, k, n):
    lib = _lib.load()
    y = torch.empty((x.shape[0], n), dtype=x.dtype, device=x.device)
    dt = _lib.F16 if x.dtype == torch.float16 else _lib.BF16
    with torch.cuda.device(x.device):
        rc = lib.exl3_linear_static(_p(x), dt, _p(packed), K, cb, _p(suh), _p(svh), _lib.int_array(ends), len(ends) + 1,
                                    x.shape[0], k, n, _p(y), dt, torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "exl3_linear_static")
    return y


@pytest.mark.parametrize("K,cb,rows,dtype", [(3, 0, 1, torch.float16), (4, 1, 5, torch.bfloat16), (5, 2, 20, torch.float16)])
def test_static_scratch_entry_point_matches_the_workspace_one(K, cb, rows, dtype):
    k, ns = 1024, [384, 256]
    n = sum(ns)
    dev = torch.device(DEV)
    _lib.init_device(0)
    trs = [torch.from_numpy(seeded_trellis(40 + i + K, k // 16, w // 16, K).view(np.int16)).to(dev) for i, w in enumerate(ns)]
    suhs = [torch.from_numpy(seeded_signs(50 + i, k)).to(dev) for i in range(2)]
    svhs = [torch.from_numpy(seeded_signs(60 + i, w)).to(dev) for i, w in enumerate(ns)]
    packed, suh_cat, svh_cat, ends = lin.prepare(trs, suhs, svhs)
    gen = torch.Generator(device=dev)
    gen.manual_seed(K * 100 + rows)
    xa = torch.randn((rows, k), device=dev, generator=gen).to(dtype)
    xb = torch.randn((rows, k), device=dev, generator=gen).to(dtype)
    want_a = lin.run(xa, packed, suh_cat, svh_cat, ends, cb)
    want_b = lin.run(xb, packed, suh_cat, svh_cat, ends, cb)
    got_a = _static_linear(xa, packed, suh_cat, svh_cat, ends, K, cb, k, n)       # first call: looks the array up
    lib, dt = _lib.load(), (_lib.F16 if dtype == torch.float16 else _lib.BF16)
    got_b = torch.empty_like(got_a)                                               # the caller's output, made before measuring
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(dev)[0]
    with torch.cuda.device(dev):                                                  # second call: reuses the array's contents
        rc = lib.exl3_linear_static(_p(xb), dt, _p(packed), K, cb, _p(suh_cat), _p(svh_cat), _lib.int_array(ends), len(ends) + 1,
                                    rows, k, n, _p(got_b), dt, torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(dev)[0] == free_before                         # the call took no device memory, from anyone
    assert torch.equal(got_a.view(torch.int16), want_a.view(torch.int16))
    assert torch.equal(got_b.view(torch.int16), want_b.view(torch.int16))
    with torch.cuda.device(dev):                                                  # no bounded wait gave up inside the static calls
        assert lib.exl3_device_error(None, 0, torch.cuda.current_stream(dev).cuda_stream) == 0


def test_static_scratch_refuses_what_does_not_fit():
    lib = _lib.load()
    assert lib.exl3_static_workspace_bytes() == 8 << 20
    k, n = 128, 128 * 2048                                          # needs far more split-k scratch than 8 MiB
    assert lib.exl3_linear_workspace_bytes(16, k, n, 1) > lib.exl3_static_workspace_bytes()
    dummy = torch.zeros(64, dtype=torch.int32, device=DEV)
    rc = lib.exl3_linear_static(_p(dummy), 0, _p(dummy), 3, 0, _p(dummy), _p(dummy), None, 1, 16, k, n, _p(dummy), 0, None)
    assert rc == 11 and b"exl3_linear_static" in lib.exl3_status_str(rc)
