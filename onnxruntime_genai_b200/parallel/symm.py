"""Symmetric peer memory for the fused GEMM + all-reduce kernel (csrc/gemm_tcgen05.cu).

Every rank owns one receive buffer `[2 parities][world sources][plane_elems / 4 lines]` of 16-byte lines
(8 payload bytes + the call's flag twice), mapped into every peer (NVLink peer access through
`torch.distributed._symmetric_memory`, which exchanges the memory handles over the process group).
The pointers are registered once with the kernel library (`ogb_comm_register`); after that the GEMM
launcher only needs a flag to run the fused path, so the call captures into CUDA graphs unchanged.

`LocalComm` registers a world of one on a single GPU: the kernel then pushes to and waits on its
own buffers, which exercises the whole protocol (parity, flagged lines, call counter) without peers.
"""
from __future__ import annotations

import ctypes
from typing import List

import torch

from ..ops import _lib

DEFAULT_PLANE_ELEMS = int(__import__("os").environ.get("OGB_COMM_PLANE_ELEMS", 2048 * 4096))  # bf16 elements per source plane of the receive buffer


def _register(device_index: int, world: int, rank: int, buf_ptrs: List[int], epoch: torch.Tensor, plane_elems: int) -> None:
    arr_t = ctypes.c_void_p * world
    rc = _lib.lib().ogb_comm_register(device_index, world, rank, arr_t(*buf_ptrs), epoch.data_ptr(), plane_elems)
    if rc != 0:
        raise RuntimeError(f"ogb_comm_register failed with {rc}")


class _Collectives:
    """Stand-alone collectives over the registered buffers (csrc/collectives.cu).  Tensors are taken as raw 16-byte
    vectors for the gather; reductions are bf16.  `fits` tells whether a tensor can go through the kernels; callers
    fall back to NCCL otherwise."""

    def fits(self, x: torch.Tensor, planes: int = 1) -> bool:
        nbytes = x.numel() * x.element_size() // planes
        return x.is_cuda and x.is_contiguous() and nbytes % 16 == 0 and nbytes // 2 <= self.plane_elems and x.data_ptr() % 16 == 0

    def _run(self, mode: int, x: torch.Tensor, out: torch.Tensor, residual, n_units: int):
        from .. import ops
        ws = ops.workspace(x.device)
        rc = _lib.lib().ogb_collective(mode, x.data_ptr(), out.data_ptr(), residual.data_ptr() if residual is not None else None,
                                       n_units, x.device.index, ws.status, ws.sm_count, torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(rc, "collective")
        return out

    def all_reduce(self, x: torch.Tensor, residual=None, out=None) -> torch.Tensor:
        """Sum over ranks (+ residual) of a bf16 tensor; every rank gets bit-identical results."""
        assert x.dtype == torch.bfloat16 and self.fits(x)
        return self._run(0, x, torch.empty_like(x) if out is None else out, residual, x.numel())

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """[world, *x.shape]: every rank's tensor, any dtype."""
        assert self.fits(x)
        out = torch.empty((self.size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        return self._run(1, x, out, None, x.numel() * x.element_size() // 2)

    def all_gather_push(self, x: torch.Tensor) -> None:
        """First half of all-gather -> GEMM: pushes this rank's token rows [rows, K] (bf16) into every rank's receive
        buffer and returns; the GEMM launched next (`ops.linear_gathered`) assembles its activation tiles from the lines
        as they arrive.  The call after that GEMM must be one that waits on every peer (any fused reduction)."""
        assert x.dtype == torch.bfloat16 and self.fits(x)
        self._run(3, x, x, None, x.numel())

    def reduce_scatter(self, x: torch.Tensor, residual=None) -> torch.Tensor:
        """x [world, ...] bf16 partials -> sum over ranks of slice [rank] (+ residual)."""
        assert x.dtype == torch.bfloat16 and x.shape[0] == self.size and self.fits(x, self.size)
        out = torch.empty(x.shape[1:], dtype=x.dtype, device=x.device)
        return self._run(2, x, out, residual, out.numel())


class LocalComm(_Collectives):
    """World of one: the fused path talking to itself (single-GPU tests of the protocol)."""

    def __init__(self, device: torch.device, plane_elems: int = DEFAULT_PLANE_ELEMS):
        self.device = device
        self.plane_elems = plane_elems
        self.rank, self.size = 0, 1
        self.max_tokens = 256
        self.buf = torch.zeros(2 * plane_elems * 2, dtype=torch.bfloat16, device=device)   # lines carry 8 of their 16 bytes as payload
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)
        _lib.init_device(device.index)
        _register(device.index, 1, 0, [self.buf.data_ptr()], self.epoch, plane_elems)

    def close(self):
        _lib.lib().ogb_comm_register(self.device.index, 0, 0, None, None, 0)


class SymmetricComm(_Collectives):
    def __init__(self, rank: int, size: int, device: torch.device, group=None, plane_elems: int = DEFAULT_PLANE_ELEMS):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.size, self.device, self.plane_elems = rank, size, device, plane_elems
        self.max_tokens = 256
        group = group or dist.group.WORLD
        self.buf = symm_mem.empty(2 * size * plane_elems * 2, dtype=torch.bfloat16, device=device)
        self.buf_h = symm_mem.rendezvous(self.buf, group)
        self.buf.zero_()     # a flag of zero never matches a call
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        _lib.init_device(device.index)
        _register(device.index, size, rank, [int(p) for p in self.buf_h.buffer_ptrs], self.epoch, plane_elems)
        dist.barrier(group=group)
