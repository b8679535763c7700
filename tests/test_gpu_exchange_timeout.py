"""Bounded waits of the tensor-parallel exchange, on ONE GPU and without any fault: the "peer" is a second region on
the same device that nobody ever writes into, so the wait for its words runs out, the kernel records that in its
error word and returns normally, the host reads the status, and the context stays usable for the next call."""
from __future__ import annotations

import ctypes

import pytest
import torch

from trellis_serve_b200 import _lib
from trellis_serve_b200.kernels import linear as lin
from trellis_serve_b200.runtime.layerset import random_packed, random_signs

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _regions(max_elems):
    lib = _lib.load()
    _lib.init_device(0)
    nbytes = int(lib.exl3_allreduce_region_bytes(max_elems))
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)     # rank 1 never runs: its words never arrive
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), silent_peer.data_ptr())
    state = torch.zeros(4, dtype=torch.int32, device=DEV)
    return mine, silent_peer, ptrs, state


def test_allreduce_gives_up_on_a_silent_peer_and_says_so():
    lib = _lib.load()
    mine, peer, ptrs, state = _regions(1024)
    x = torch.ones(64, dtype=torch.float16, device=DEV)
    st = torch.cuda.current_stream(DEV).cuda_stream
    with torch.cuda.device(DEV):
        _lib.check(lib.exl3_allreduce(ctypes.c_void_p(x.data_ptr()), _lib.F16, 64, ptrs, 0, 2, 1024, ctypes.c_void_p(state.data_ptr()), st),
                   "exl3_allreduce")
    torch.cuda.synchronize()                                             # the kernel ended by itself
    assert int(state[1].item()) != 0                                     # ... and recorded that a peer did not arrive
    assert int(state[0].item()) == 1                                     # the call still counts: ranks stay in step
    # the context is intact: a world of one on the same stream works
    y = torch.full((64,), 3.0, dtype=torch.float16, device=DEV)
    with torch.cuda.device(DEV):
        _lib.check(lib.exl3_allreduce(ctypes.c_void_p(y.data_ptr()), _lib.F16, 64, ptrs, 0, 1, 1024, ctypes.c_void_p(state.data_ptr()), st),
                   "exl3_allreduce")
    torch.cuda.synchronize()
    assert torch.all(y == 3.0)


def test_fused_linear_gives_up_on_a_silent_peer_and_reports_a_device_wait():
    gen = torch.Generator(device=DEV)
    gen.manual_seed(5)
    k, n, K = 256, 512, 3
    w = random_packed(k, n, K, gen, DEV)
    suh, svh = random_signs(k, gen, DEV, 1), random_signs(n, gen, DEV).view(-1)
    x = torch.randn((1, k), device=DEV, generator=gen).half()
    mine, peer, ptrs, state = _regions(16 * n)

    class SilentPeerExchange:                                            # the fields kernels.linear.run reads
        world, rank, max_elems, peer_regions = 2, 0, 16 * n, ptrs
    SilentPeerExchange.state = state
    want = lin.run(x, w, suh, svh, [], 0)
    lin.run(x, w, suh, svh, [], 0, exchange=SilentPeerExchange)
    torch.cuda.synchronize()
    with pytest.raises(_lib.Exl3Error) as e:
        lin.device_error(DEV)                                            # reads and clears the error word
    assert "wait" in str(e.value).lower()
    lin.device_error(DEV)                                                # cleared
    assert torch.equal(lin.run(x, w, suh, svh, [], 0), want)             # the library keeps working
