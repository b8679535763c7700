"""Exchange step of row-parallel EXL3 linears: a one-shot all-reduce over peer-mapped memory.

`PeerAllReduce` owns one symmetric region per rank (allocated and exchanged through torch's symmetric-memory
rendezvous: plumbing only) and calls `exl3_allreduce` (csrc/exl3_allreduce.cu), the library's own kernel: every rank
pushes its values into its slot at every peer with ordinary peer stores over NVLink, each 32-bit pair of values in one
64-bit word together with the call number, then polls its OWN memory (bounded) until the words of every rank carry that
call number and adds them in rank order in fp32.  No flags, no fences, no peer loads, no multicast; every rank gets the
same bits.  `exl3_linear_allreduce` runs the same protocol inside the epilogue of a row-parallel linear.
`nccl_all_reduce` is the library-collective alternative, kept for comparison.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _lib


def nccl_all_reduce(t: torch.Tensor, group=None) -> torch.Tensor:
    dist.all_reduce(t, group=group)
    return t


class PeerAllReduce:
    """In-place sum of fp16 / bf16 tensors of up to `max_elems` elements over the ranks of `group` (one node)."""

    def __init__(self, device: torch.device, max_elems: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device, self.max_elems = torch.device(device), int(max_elems)
        lib = _lib.load()
        _lib.init_device(self.device.index)
        nbytes = int(lib.exl3_allreduce_region_bytes(self.max_elems))
        self.region = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.region.zero_()
        self.handle = symm_mem.rendezvous(self.region, self.group.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.world:
            raise RuntimeError(f"symmetric-memory rendezvous returned {len(ptrs)} peers for a group of {self.world}")
        self.peer_regions = (ctypes.c_void_p * self.world)(*ptrs)
        self.state = torch.zeros(4, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)                 # every region is zero before anyone stores into a peer

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        if t.dtype not in (torch.float16, torch.bfloat16) or not t.is_contiguous():
            raise TypeError("PeerAllReduce takes contiguous fp16 / bf16 tensors")
        code = _lib.F16 if t.dtype == torch.float16 else _lib.BF16
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().exl3_allreduce(ctypes.c_void_p(t.data_ptr()), code, t.numel(), self.peer_regions, self.rank,
                                                  self.world, self.max_elems, ctypes.c_void_p(self.state.data_ptr()),
                                                  torch.cuda.current_stream(self.device).cuda_stream), "exl3_allreduce")
        return t

    def check(self) -> None:
        """Raises if a bounded wait for a peer gave up since the last check (synchronises)."""
        code = int(self.state[1].item())
        if code:
            self.state[1] = 0
            raise _lib.Exl3Error(7, "exl3_allreduce", f"a peer did not arrive in time (device code {code})")
