"""Symmetric peer memory for the fused GEMM + all-reduce kernel (csrc/gemm_tcgen05.cu).

Every rank owns one receive buffer `[2 parities][world sources][plane_elems]` bf16 and one array of
arrival counters; both are mapped into every peer (NVLink peer access through
`torch.distributed._symmetric_memory`, which exchanges the memory handles over the process group).
The pointers are registered once with the kernel library (`ogb_comm_register`); after that the GEMM
launcher only needs a flag to run the fused path, so the call captures into CUDA graphs unchanged.

`LocalComm` registers a world of one on a single GPU: the kernel then pushes to and waits on its
own buffers, which exercises the whole protocol (parity, counters, use counts) without peers.
"""
from __future__ import annotations

import ctypes
from typing import List

import torch

from ..ops import _lib

MAX_SLOTS = 4096
DEFAULT_PLANE_ELEMS = 256 * 8192  # up to 256 tokens x 8192 output features per fused call


def _register(device_index: int, world: int, rank: int, buf_ptrs: List[int], flag_ptrs: List[int], uses: torch.Tensor,
              plane_elems: int) -> None:
    arr_t = ctypes.c_void_p * world
    rc = _lib.lib().ogb_comm_register(device_index, world, rank, arr_t(*buf_ptrs), arr_t(*flag_ptrs), uses.data_ptr(),
                                      plane_elems, MAX_SLOTS)
    if rc != 0:
        raise RuntimeError(f"ogb_comm_register failed with {rc}")


class LocalComm:
    """World of one: the fused path talking to itself (single-GPU tests of the protocol)."""

    def __init__(self, device: torch.device, plane_elems: int = DEFAULT_PLANE_ELEMS):
        self.device = device
        self.plane_elems = plane_elems
        self.max_tokens = 256
        self.buf = torch.zeros(2 * plane_elems, dtype=torch.bfloat16, device=device)
        self.flags = torch.zeros(MAX_SLOTS, dtype=torch.int32, device=device)
        self.uses = torch.zeros(MAX_SLOTS, dtype=torch.int32, device=device)
        _lib.init_device(device.index)
        _register(device.index, 1, 0, [self.buf.data_ptr()], [self.flags.data_ptr()], self.uses, plane_elems)

    def close(self):
        _lib.lib().ogb_comm_register(self.device.index, 0, 0, None, None, None, 0, 0)


class SymmetricComm:
    def __init__(self, rank: int, size: int, device: torch.device, group=None, plane_elems: int = DEFAULT_PLANE_ELEMS):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.size, self.device, self.plane_elems = rank, size, device, plane_elems
        self.max_tokens = 256
        group = group or dist.group.WORLD
        self.buf = symm_mem.empty(2 * size * plane_elems, dtype=torch.bfloat16, device=device)
        self.flags = symm_mem.empty(MAX_SLOTS, dtype=torch.int32, device=device)
        self.buf_h = symm_mem.rendezvous(self.buf, group)
        self.flag_h = symm_mem.rendezvous(self.flags, group)
        self.flags.zero_()
        self.uses = torch.zeros(MAX_SLOTS, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        _lib.init_device(device.index)
        _register(device.index, size, rank, [int(p) for p in self.buf_h.buffer_ptrs], [int(p) for p in self.flag_h.buffer_ptrs],
                  self.uses, plane_elems)
        dist.barrier(group=group)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Stand-alone all-reduce for tensors that did not come out of a fused GEMM (NCCL)."""
        import torch.distributed as dist
        dist.all_reduce(x)
        return x
